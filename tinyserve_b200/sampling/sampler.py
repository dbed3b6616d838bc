"""Batched sampling on the device: one call for rows with mixed settings.

Order as in tinyserve's ``sample`` (serve.py:1501-1588): repetition penalty on the
logits, then argmax for greedy rows, else temperature, top-k, top-p and Gumbel-max.
Unlike there, the noise of a row depends only on (engine seed, the request's stream,
how many tokens the request has generated), not on the batch around it."""
from __future__ import annotations

import zlib

import torch

from ..kernels import ops


def stream_of(request_id, params) -> int:
    """The request's noise stream: its ``seed`` if given, else a hash of its id."""
    if params.seed is not None:
        return int(params.seed) & (2 ** 63 - 1)
    return zlib.crc32(str(request_id).encode()) | (1 << 40)


def recent_tokens(params, token_ids) -> list:
    """Distinct tokens the repetition penalty applies to (serve.py:1469-1476)."""
    if params.repetition_penalty == 1.0 or params.repeat_last_n == 0:
        return []
    window = token_ids if params.repeat_last_n < 0 else token_ids[-params.repeat_last_n:]
    return sorted(set(window))


class Sampler:
    def __init__(self, seed: int, device, max_rows: int = 0):
        self.seed = int(seed)
        self.device = device
        self._zeros: dict = {}
        self._staging = None
        self._rows = max_rows
        self._flip = 0

    def _settings(self, temps, ks, ps, streams, steps):
        """The per-row settings as device tensors, through one pinned staging buffer and one copy
        (two buffers take turns: the copy of the step before may still be pending)."""
        n = len(temps)
        if self._staging is None or n > self._rows:
            self._rows = max(self._rows, n, 8)
            words = 6 * self._rows                    # float32 temp, float32 top_p, int32 top_k, int32 steps, int64 streams
            pin = torch.device(self.device).type == "cuda"
            self._staging = [(torch.zeros(words, dtype=torch.int32).pin_memory() if pin
                              else torch.zeros(words, dtype=torch.int32)) for _ in range(2)]
            self._device_words = torch.zeros(words, dtype=torch.int32, device=self.device)
        R = self._rows
        host = self._staging[self._flip]
        self._flip ^= 1
        h = host.numpy()
        h[0:n].view("float32")[:] = temps
        h[R:R + n].view("float32")[:] = ps
        h[2 * R:2 * R + n] = ks
        h[3 * R:3 * R + n] = steps
        h[4 * R:4 * R + 2 * n].view("int64")[:] = streams
        d = self._device_words
        d.copy_(host, non_blocking=True)
        return (d[0:n].view(torch.float32), d[R:R + n].view(torch.float32), d[2 * R:2 * R + n],
                d[3 * R:3 * R + n], d[4 * R:4 * R + 2 * n].view(torch.int64))

    def _greedy_args(self, n):
        """Device tensors for an all-greedy batch (temperature 0 ignores the noise arguments)."""
        if n not in self._zeros:
            self._zeros[n] = (torch.zeros(n, dtype=torch.float32, device=self.device),
                              torch.zeros(n, dtype=torch.int64, device=self.device),
                              torch.zeros(n, dtype=torch.int32, device=self.device))
        return self._zeros[n]

    def __call__(self, logits, requests, slot_tokens=None, slots=None):
        """logits float32 [B, V] (modified in place by the penalty); ``requests``: objects with
        request_id, params, token_ids, prompt_len.  Returns int32 [B] on the device.  With
        ``slot_tokens`` and ``slots`` (int32 [B], device) every token is also left at its request's
        state slot for the next step."""
        B = logits.shape[0]
        feedback = dict(slot_tokens=slot_tokens, slots=slots)
        if all(r.params.temperature == 0 and (r.params.repetition_penalty == 1.0 or r.params.repeat_last_n == 0)
               for r in requests):
            temps, streams, steps = self._greedy_args(B)
            return ops.sample(logits, temps, streams, steps, self.seed, **feedback)
        temps, ks, ps, streams, steps = [], [], [], [], []
        pen_rows, pen_ids, pen_vals = [], [], []
        for i, r in enumerate(requests):
            p = r.params
            temps.append(float(p.temperature))
            ks.append(int(p.top_k) if p.top_k and p.top_k > 0 else 0)
            ps.append(float(p.top_p))
            streams.append(stream_of(r.request_id, p))
            steps.append(len(r.token_ids) - r.prompt_len)
            ids = recent_tokens(p, r.token_ids)
            if ids:
                pen_rows.append(i)
                pen_ids.append(ids)
                pen_vals.append(float(p.repetition_penalty))
        dev = self.device
        if pen_rows:
            width = max(len(x) for x in pen_ids)
            table = torch.full((len(pen_rows), width), -1, dtype=torch.int32)
            for j, ids in enumerate(pen_ids):
                table[j, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
            ops.apply_repetition_penalty(logits, torch.tensor(pen_rows, dtype=torch.int32, device=dev),
                                         table.to(dev), torch.tensor(pen_vals, dtype=torch.float32, device=dev))
        need_k = any(k > 0 for k, t in zip(ks, temps) if t > 0)
        need_p = any(p < 1.0 for p, t in zip(ps, temps) if t > 0)
        d_temps, d_ps, d_ks, d_steps, d_streams = self._settings(temps, ks, ps, streams, steps)
        return ops.sample(logits, d_temps, d_streams, d_steps, self.seed, top_k=d_ks if need_k else None,
                          top_p=d_ps if need_p else None, **feedback)
