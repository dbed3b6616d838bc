"""The status words that kernels write when they give up on a bounded wait or (in a
bounds-checking build) meet an index out of range: a set word stops the engine with a message."""
import pytest


def test_a_status_code_raises_and_names_its_reason():
    from tinyserve_b200.kernels import ops
    words = ops.status_words()
    assert not words.any()
    ops.raise_on_device_error()
    try:
        words[0] = 1
        with pytest.raises(ops.DeviceError, match="bounded wait"):
            ops.raise_on_device_error()
        words[0] = 0
        words[1] = 2
        with pytest.raises(ops.DeviceError, match="cache slot"):
            ops.raise_on_device_error()
        words[1] = 99
        with pytest.raises(ops.DeviceError, match="out of range"):
            ops.raise_on_device_error()
    finally:
        words[:] = 0
    ops.raise_on_device_error()
