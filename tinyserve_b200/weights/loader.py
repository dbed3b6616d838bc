"""Weights from safetensors, by tensor name.

The model's parts declare what they need (``ParamSpec``); this module turns that
into the list of checkpoint tensors, reads them from every ``*.safetensors`` of the
folder (sorted, as serve.py:1389-1393 does; the index json is not needed), places
fused parameters row range by row range (q/k/v into qkv_proj, gate/up into
gate_up_proj: serve.py:72-74, 1352-1358) and hands every part its tensors.

Dtypes: matrices are kept in the engine's dtype; vectors too, except that a tensor
the file stores in 32-bit stays 32-bit; integer tables become int32.

Errors: one ``WeightError`` lists all missing tensors, all unexpected tensors and all
wrong shapes (tinyserve asserts on missing ones and warns on unused ones,
serve.py:1397-1403).  ``lm_head.weight`` in a checkpoint of a tied model is ignored,
as it has no home there either (serve.py:1385-1387)."""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
from safetensors import safe_open

from ..parts.base import ParamSpec, Source, interleave_halves


class WeightError(RuntimeError):
    """The checkpoint does not fit the model; the message lists every fault."""

    def __init__(self, missing, unexpected, wrong_shape, duplicates=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.duplicates = list(wrong_shape), list(duplicates)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        if self.duplicates:
            lines.append(f"  stored twice ({len(self.duplicates)}): " + ", ".join(self.duplicates))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class ExpectedTensor:
    name: str            # checkpoint tensor name
    shape: tuple
    part: object
    param: str           # local parameter name in the part
    spec: ParamSpec
    row_start: int
    row_end: int


def _sources(local_name: str, spec: ParamSpec):
    if spec.sources:
        return spec.sources
    rows = spec.shape[0] if spec.shape else 1
    return (Source(local_name, 0, rows),)


def expected_tensors(model) -> list:
    """Every checkpoint tensor the model reads, in a fixed order."""
    out = []
    for part in model.named_parts():
        for local, spec in part.param_specs().items():
            for src in _sources(local, spec):
                shape = (src.row_end - src.row_start,) + tuple(spec.shape[1:])
                out.append(ExpectedTensor(f"{part.path}.{src.name}", shape, part, local, spec,
                                          src.row_start, src.row_end))
    return out


def _param_dtype(spec: ParamSpec, engine_dtype, stored_dtypes):
    if spec.role == "int_table":
        return torch.int32
    if spec.role == "vector" and all(d == torch.float32 for d in stored_dtypes):
        return torch.float32
    return engine_dtype


def _index_folder(model_dir):
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"{model_dir!r} holds no *.safetensors file")
    index, duplicates = {}, []
    for fname in files:
        with safe_open(os.path.join(model_dir, fname), "pt", device="cpu") as fh:
            for key in fh.keys():
                if key in index:
                    duplicates.append(key)
                sl = fh.get_slice(key)
                index[key] = (fname, tuple(sl.get_shape()), sl.get_dtype())
    return index, duplicates


_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "F64": torch.float64, "I32": torch.int32, "I64": torch.int64, "I16": torch.int16,
              "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}


def check_checkpoint(model, index, duplicates=()):
    """Compare the model's expected tensors with a {name: (file, shape, dtype)} index."""
    expected = expected_tensors(model)
    names = {e.name for e in expected}
    missing = [e.name for e in expected if e.name not in index]
    tied = model.lm_head is None if hasattr(model, "lm_head") else False
    unexpected = [k for k in sorted(index) if k not in names
                  and not (tied and k == "lm_head.weight")]
    wrong = [(e.name, index[e.name][1], e.shape) for e in expected
             if e.name in index and tuple(index[e.name][1]) != tuple(e.shape)]
    if missing or unexpected or wrong or duplicates:
        raise WeightError(missing, unexpected, wrong, duplicates)
    return expected


def load_weights(model, model_dir: str, dtype: torch.dtype, device) -> int:
    """Fill every part of ``model`` from ``model_dir``; returns the bytes placed."""
    index, duplicates = _index_folder(model_dir)
    expected = check_checkpoint(model, index, duplicates)
    by_param = {}
    for e in expected:
        by_param.setdefault((id(e.part), e.param), []).append(e)
    tensors, handles, total = {}, {}, 0
    try:
        for (_, local), entries in by_param.items():
            part, spec = entries[0].part, entries[0].spec
            stored = [_ST_DTYPES.get(index[e.name][2], torch.float32) for e in entries]
            pdtype = _param_dtype(spec, dtype, stored)
            param = torch.empty(spec.shape, dtype=pdtype, device=device)
            for e in entries:
                fname = index[e.name][0]
                if fname not in handles:
                    handles[fname] = safe_open(os.path.join(model_dir, fname), "pt", device="cpu")
                src = handles[fname].get_tensor(e.name)
                dst = param[e.row_start:e.row_end] if param.dim() else param
                dst.copy_(src.to(pdtype) if src.dtype != pdtype else src)
            if spec.interleave_halves:
                param = interleave_halves(param, spec.interleave_halves).contiguous()
            tensors.setdefault(id(part), (part, {}))[1][local] = param
            total += param.numel() * param.element_size()
    finally:
        handles.clear()
    for part, bound in tensors.values():
        part.bind(bound)
    for part in model.named_parts():
        if id(part) not in tensors:
            part.bind({})
    return total
