"""The allocation-free tensor-core matmul entry point (mk_k_q4k_matmul_tc_noalloc_dev).

It serves hosts that own all GPU memory themselves and may not let a library allocate on the request
path (a serving process with its own device arena, a sandboxed plugin).  The caller hands in device
pointers; the kernel's working storage is a fixed device array inside the library.  This test calls it
through the C ABI twice in a row - the second call reuses the arrays the first one dirtied - and checks
each result against the ordinary entry point (mk_k_qmatmul on the tensor-core path), which allocates
its scratch.  It lives in a file pytest collects last, so a failure here cannot hide other tests.
"""
import ctypes as C
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(mk):
    torch = pytest.importorskip("torch")
    capi = importlib.import_module("macllm_infer_b200._capi")
    ops = importlib.import_module("macllm_infer_b200.ops")
    if capi.lib().mk_device_count() <= 0:
        pytest.fail("this test needs a CUDA device: the library has no CPU fallback")
    return torch, capi, ops


def call_noalloc(torch, capi, w_bytes, rows, cols, x):
    """Device buffers come from torch (the stand-in for a host that owns the arena); the library
    receives raw device pointers only."""
    dev = torch.device("cuda", 0)
    w_dev = torch.from_numpy(np.ascontiguousarray(w_bytes)).to(dev)
    x_dev = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(dev)
    y_dev = torch.full((x.shape[0], rows), float("nan"), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    status = capi.lib().mk_k_q4k_matmul_tc_noalloc_dev(C.c_void_p(w_dev.data_ptr()), rows, cols, C.c_void_p(x_dev.data_ptr()),
                                                      x.shape[0], C.c_void_p(y_dev.data_ptr()), None)
    capi.check(status)
    free_after, _ = torch.cuda.mem_get_info()
    return y_dev.cpu().numpy(), free_before - free_after


def test_two_calls_in_a_row_match_the_allocating_entry_point(env):
    torch, capi, ops = env
    rng = np.random.default_rng(11)
    # different shapes on purpose: the second call must not see anything the first one left behind
    cases = [(40, 768, 2048, 5), (64, 2048, 1024, 6)]
    for call, (T, rows, cols, stream) in enumerate(cases):
        w = ops.seed_tensor(0, stream, 0.02, capi.TYPE_Q4_K, rows, cols)
        x = rng.standard_normal((T, cols)).astype(np.float32)
        want = ops.qmatmul(capi.TYPE_Q4_K, w, rows, cols, x, capi.PATH_TENSOR)
        got, taken = call_noalloc(torch, capi, w, rows, cols, x)
        assert np.isfinite(got).all()
        # the first call on a device may load the library's kernels (module loading is lazy); from the second call
        # on, the device's free memory is the same before and after: nothing was allocated
        if call > 0:
            assert taken == 0
        # same kernels, same operands, same split order: the tolerance of the tensor-core tests, and in
        # practice bit-identical
        scale = np.sqrt(cols) * 0.02
        assert np.max(np.abs(got - want)) <= 2e-3 * scale
        assert np.max(np.abs(got - want)) <= 1e-6


def test_sizes_beyond_the_built_in_scratch_are_refused(env):
    torch, capi, ops = env
    dev = torch.device("cuda", 0)
    rows, cols, T = 256, 8192, 128  # T * cols = 1 Mi elements > 512 Ki
    w_dev = torch.zeros(rows * (cols // 256) * 144, dtype=torch.uint8, device=dev)
    x_dev = torch.zeros((T, cols), dtype=torch.float32, device=dev)
    y_dev = torch.zeros((T, rows), dtype=torch.float32, device=dev)
    status = capi.lib().mk_k_q4k_matmul_tc_noalloc_dev(C.c_void_p(w_dev.data_ptr()), rows, cols, C.c_void_p(x_dev.data_ptr()), T,
                                                      C.c_void_p(y_dev.data_ptr()), None)
    assert status < 0
    assert b"exceeds the built-in activation scratch" in capi.lib().mk_last_error()
    # a bad shape is refused before anything runs
    status = capi.lib().mk_k_q4k_matmul_tc_noalloc_dev(C.c_void_p(w_dev.data_ptr()), rows, 100, C.c_void_p(x_dev.data_ptr()), 1,
                                                      C.c_void_p(y_dev.data_ptr()), None)
    assert status < 0
