"""fp8_gemm without any device allocation: `dsv3_fp8_gemm_static` against `dsv3_fp8_gemm`.

Some hosts cannot give the library a split-K workspace: a serving process that has already committed
the whole GPU to its own arena cannot afford a cudaMalloc while requests are in flight (it may fail, and
it stalls every stream while the driver synchronises the device), and a plain C program has no framework
allocator to borrow from.  For them the library carries a fixed scratch array inside its image.  This test
drives that entry point through the C ABI with raw pointers, twice in a row on different problems (the
array keeps what the previous call left behind), and expects the very same bf16 bits the regular entry
point produces with a caller-provided workspace -- both run the same kernel with the same deterministic
split-K reduction.  It also checks that free device memory does not move across the calls and that a
problem too large for the array is refused instead of overrunning it.

The file sorts last on purpose: a failure here cannot hide the result of any other test in a run that
stops at the first failure.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O
from gpu_util import bf16_bits, assert_gemm_close

pytestmark = pytest.mark.gpu


def _quantised(M, N, K, seed):
    x, _, wq, ws = O.make_case(M, N, K, seed)
    xq, xs = O.act_quant(x)
    return xq.cuda(), xs.cuda(), wq.cuda(), ws.cuda()


def _regular(lib, _lib, xq, xs, wq, ws, M, N, K):
    """The existing entry point with a workspace allocated by the caller (torch)."""
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    need = lib.dsv3_fp8_gemm_workspace_bytes(M, N, K)
    ws_buf = torch.zeros(max(need, 1), dtype=torch.uint8, device="cuda")
    _lib.check(lib.dsv3_fp8_gemm(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, N, K, c.data_ptr(),
                                 ws_buf.data_ptr(), ws_buf.numel(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return c, need


def _static(lib, _lib, xq, xs, wq, ws, M, N, K):
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.dsv3_fp8_gemm_static(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, N, K,
                                        c.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return c


def test_static_scratch_gemm_matches_regular_entry_point_twice_in_a_row():
    from dsv3_b200 import _lib
    lib = _lib.lib
    _lib.check(lib.dsv3_set_gemm_policy(0, 0))
    assert lib.dsv3_fp8_gemm_static_scratch_bytes() >= _lib.WORKSPACE_HEADER_BYTES + (1 << 20)
    # two decode-sized problems that split K (few output tiles), then one that does not
    problems = [(32, 1024, 4096, 51), (8, 576, 7168, 52), (300, 2048, 512, 53)]
    inputs = [(_quantised(*p), p) for p in problems]
    # references first, so that every torch allocation is done before free memory is sampled
    refs = [_regular(lib, _lib, *t, *p[:3]) for t, p in inputs]
    assert refs[0][1] > 0 and refs[1][1] > 0, "the first two problems are meant to use split-K scratch"
    outs = [torch.empty(p[0], p[1], dtype=torch.bfloat16, device="cuda") for _, p in inputs]
    stream = torch.cuda.current_stream().cuda_stream
    # first call on this device resolves the array's address; do it before sampling free memory
    t, p = inputs[0]
    _lib.check(lib.dsv3_fp8_gemm_static(*(v.data_ptr() for v in t), *p[:3], outs[0].data_ptr(), stream))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for round_ in range(2):                       # "two calls in a row", and once more over all problems
        for (t, p), out in zip(inputs, outs):
            out.zero_()
            _lib.check(lib.dsv3_fp8_gemm_static(*(v.data_ptr() for v in t), *p[:3], out.data_ptr(), stream))
        torch.cuda.synchronize()
        for (ref, _), out, (t, p) in zip(refs, outs, inputs):
            assert np.array_equal(bf16_bits(out), bf16_bits(ref)), f"round {round_}, problem {p[:3]}"
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the static entry point must not allocate device memory"
    # and the result is right in the first place: against the CPU oracle, stated fp8_gemm tolerance
    (xq, xs, wq, ws), p = inputs[0]
    assert_gemm_close(outs[0], O.fp8_gemm(xq.cpu(), xs.cpu(), wq.cpu(), ws.cpu()))
    detail = (ctypes.c_uint32 * 4)()
    assert lib.dsv3_check_device_status(stream, ctypes.byref(detail)) == _lib.OK


def test_static_scratch_gemm_uses_fewer_splits_when_the_automatic_plan_does_not_fit():
    from dsv3_b200 import _lib
    lib = _lib.lib
    _lib.check(lib.dsv3_set_gemm_policy(0, 0))
    M, N, K = 384, 3072, 7168        # 72 tiles of 128 x 128: the automatic plan splits K in two, 9.4 MB of partial tiles
    xq, xs, wq, ws = _quantised(M, N, K, 55)
    ref, need = _regular(lib, _lib, xq, xs, wq, ws, M, N, K)
    if need <= lib.dsv3_fp8_gemm_static_scratch_bytes():
        pytest.skip("the automatic plan of this problem fits the array on this device")
    out = _static(lib, _lib, xq, xs, wq, ws, M, N, K)
    assert_gemm_close(out, ref.cpu())
    assert_gemm_close(out, O.fp8_gemm(xq.cpu(), xs.cpu(), wq.cpu(), ws.cpu()))


def test_static_scratch_gemm_refuses_what_does_not_fit():
    from dsv3_b200 import _lib
    lib = _lib.lib
    M, N, K = 1024, 1024, 2048
    xq, xs, wq, ws = _quantised(M, N, K, 54)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    try:
        _lib.check(lib.dsv3_set_gemm_policy(2, 8))     # 8 splits x 4 MiB of partial sums > the array
        assert lib.dsv3_fp8_gemm_workspace_bytes(M, N, K) > lib.dsv3_fp8_gemm_static_scratch_bytes()
        rc = lib.dsv3_fp8_gemm_static(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), M, N, K,
                                      c.data_ptr(), stream)
        assert rc == _lib.ERR_WORKSPACE
        assert b"built-in array" in lib.dsv3_last_error()
    finally:
        _lib.check(lib.dsv3_set_gemm_policy(0, 0))
    # shapes outside the tcgen05 kernels' limits are refused as well (no silent other path)
    xq2, xs2, wq2, ws2 = (t.cuda() for t in (torch.zeros(4, 100, dtype=torch.uint8), torch.ones(4, 1),
                                             torch.zeros(64, 100, dtype=torch.uint8), torch.ones(1, 1)))
    c2 = torch.empty(4, 64, dtype=torch.bfloat16, device="cuda")
    rc = lib.dsv3_fp8_gemm_static(xq2.data_ptr(), xs2.data_ptr(), wq2.data_ptr(), ws2.data_ptr(), 4, 64, 100,
                                  c2.data_ptr(), stream)
    assert rc == _lib.ERR_UNSUPPORTED
    assert lib.dsv3_fp8_gemm_static(None, None, None, None, 0, 64, 128, None, stream) == _lib.OK
