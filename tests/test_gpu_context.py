"""GPU tests of the context's bookkeeping through the C ABI: the weight stack and the weight arena, what is refused
while a command batch is being recorded, and that a failed registration leaves the arena as it found it."""
import ctypes as C

import numpy as np
import pytest

from helpers import register
from webllm_b200 import Gpu, QwenGpt, WebllmError, _lib, synthetic

pytestmark = pytest.mark.gpu

TINY = synthetic.QwenShape(97, 1, 4, 2, 128, 128)


def test_weight_pop_is_refused_once_a_model_carved_the_arena(built_lib):
    """A model takes its KV cache and decode buffers from the weight arena after the weights: popping a weight then
    would hand that memory to the next registration. Destroying the model returns its carve and the pop works again."""
    with Gpu(0, weight_bytes=64 << 20, act_bytes=16 << 20) as gpu:
        model = QwenGpt(gpu, TINY, max_t=32)
        model.upload_gptq_model(synthetic.random_qwen_gptq(TINY, seed=1), fuse=True)
        weights_top = Arena_used(gpu)
        model.prefill(np.array([1, 2, 3], np.uint32), last_only=True)  # creates the device-side model (the carve)
        assert Arena_used(gpu) > weights_top
        with pytest.raises(WebllmError) as e:
            gpu.weight_pop()
        assert e.value.status == _lib.WB_ERR_BAD_ARG and "cannot be dropped" in str(e.value)
        model.close()
        assert Arena_used(gpu) == weights_top  # the carve came back
        gpu.weight_pop()
        assert Arena_used(gpu) < weights_top


def Arena_used(gpu) -> int:
    from webllm_b200.device import Arena
    return Arena(gpu, _lib.WB_ARENA_WEIGHTS).used_bytes


def test_failed_registration_rolls_the_arena_back(built_lib):
    """qweight fits, the scales do not: the registration fails with WB_ERR_OOM and the piece it had already taken is
    handed back, so a smaller weight still finds the whole arena."""
    t = synthetic.random_gptq(1024, 256, 128, seed=2)          # qweight 128 KiB, scales 4 KiB, zeros 1 KiB
    with Gpu(0, weight_bytes=(128 << 10) + 2048, act_bytes=1 << 20) as gpu:
        before = Arena_used(gpu)
        with pytest.raises(WebllmError) as e:
            register(gpu, "too_big", t)
        assert e.value.status == _lib.WB_ERR_OOM
        assert Arena_used(gpu) == before
        small = synthetic.random_gptq(256, 64, 128, seed=3)
        register(gpu, "fits", small)
        with pytest.raises(WebllmError):
            gpu.weight("too_big")


def test_blocking_calls_are_refused_while_recording(gpu):
    """Transfers, registrations and synchronize would fail inside CUDA on a capturing stream and invalidate the
    recording; they are refused up front with the rule in the message and the recording stays usable."""
    t = synthetic.random_gptq(256, 64, 128, seed=4)
    h = register(gpu, "rec_w", t)
    gpu.arena.reset()
    A, Y = gpu.arena.alloc(256), gpu.arena.alloc(64)
    gpu.write(A, np.ones(256, np.float32))
    with gpu.batch() as b:
        gpu.linear(h, A, Y, None, 1)
        for call in (lambda: gpu.write(A, np.zeros(256, np.float32)), lambda: gpu.read(Y), gpu.synchronize,
                     lambda: register(gpu, "rec_w2", t), lambda: gpu.f32_upload("rec_b", np.zeros(4, np.float32)),
                     gpu.weight_pop):
            with pytest.raises(WebllmError, match="while a command batch is being recorded") as e:
                call()
            assert e.value.status == _lib.WB_ERR_BAD_ARG
    b.submit()
    first = gpu.read(Y)
    b.submit()
    assert np.array_equal(first, gpu.read(Y)) and np.any(first != 0)
    b.destroy()
