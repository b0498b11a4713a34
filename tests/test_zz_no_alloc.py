"""The allocation-free entry point of the tensor-core matrix product, called the way its
users call it: through the exported C symbol of the shared library, with raw device pointers.

Who needs it: callers that may not allocate device memory, because they run while a graph
is being captured, sit in a loop where an allocation would stall the device, or live in a
host process that owns all device memory.  The split-K scratch is a fixed array inside the
library; this test checks that two calls in a row give what the ordinary entry point gives
(the second call finds the first call's partial sums in the array and must not be disturbed
by them), that a product of a few hundred tokens, which keeps a partial tile per block in the
scratch, and one of 512 tokens, which cuts K into ranges on pairs of blocks, stay within the
array, that a product whose plan needs more than the array is refused before anything is
launched, and that the free device memory is the same before and after a call."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def static_entry():
    from spyinfer_b200.csrc import build
    lib = build.load("gemm_tcgen05")
    fn = lib.spy_gemm_tcgen05_static_scratch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    err = lib.spy_gemm_tcgen05_last_error
    err.restype = ctypes.c_char_p
    return fn, err


def test_static_scratch_entry_matches_the_ordinary_one_twice_in_a_row():
    from spyinfer_b200 import kernels
    fn, err = static_entry()
    status = kernels.status_word(DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # both shapes split K (few output tiles); the second is smaller, so stale partial sums of
    # the first call lie around and beyond the region the second call uses
    for seed, (M, N, K) in enumerate([(24, 1024, 4096), (5, 384, 2048)]):
        torch.manual_seed(seed)
        a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
        want = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        kernels.gemm_tcgen05(a, w, want)
        got = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        rc = fn(a.data_ptr(), K, w.data_ptr(), K, got.data_ptr(), 1, N, M, N, K, status.data_ptr(), stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        assert status[0].item() == 0
        torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=2e-3)
        ref = (a.float() @ w.float().t()).to(torch.bfloat16).float()
        torch.testing.assert_close(got.float(), ref, rtol=1.6e-2, atol=2e-3)


def test_static_scratch_entry_shares_a_few_hundred_tokens_within_its_array():
    """A product with fewer tiles than SMs shares its K blocks out over the SMs and keeps a partial
    tile per block in the scratch; the built-in array (4 Mi floats) holds 128 of them, so the entry
    point uses at most 128 blocks and gives the product all the same, twice in a row."""
    fn, err = static_entry()
    M, N, K = 300, 4096, 8192           # 3 x 16 tiles of 128 x 256
    torch.manual_seed(3)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = (a.float() @ w.float().t()).to(torch.bfloat16).float()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        rc = fn(a.data_ptr(), K, w.data_ptr(), K, out.data_ptr(), 1, N, M, N, K, None, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), ref, rtol=1.6e-2, atol=2e-3)


def test_static_scratch_entry_cuts_k_into_ranges_within_its_array_and_allocates_nothing():
    """512 tokens on 32 tiles of 256 x 256: K is cut into two ranges on pairs of blocks, whose
    partial products (2 x 512 x 4096 floats) fill the array exactly.  The first call may load the
    kernel's code onto the device; from then on the free device memory does not move across a call."""
    fn, err = static_entry()
    M, N, K = 512, 4096, 4096
    torch.manual_seed(4)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    ref = (a.float() @ w.float().t()).to(torch.bfloat16).float()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = [torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    small = [torch.randn(24, 4096, device=DEV).to(torch.bfloat16), torch.randn(1024, 4096, device=DEV).to(torch.bfloat16) / 64,
             torch.empty(24, 1024, device=DEV, dtype=torch.bfloat16)]
    assert fn(a.data_ptr(), K, w.data_ptr(), K, outs[0].data_ptr(), 1, N, M, N, K, None, stream) == 0, err().decode()
    assert fn(small[0].data_ptr(), 4096, small[1].data_ptr(), 4096, small[2].data_ptr(), 1, 1024, 24, 1024, 4096, None, stream) == 0, err().decode()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(DEV)[0]
    for out in outs[1:]:
        assert fn(a.data_ptr(), K, w.data_ptr(), K, out.data_ptr(), 1, N, M, N, K, None, stream) == 0, err().decode()
    assert fn(small[0].data_ptr(), 4096, small[1].data_ptr(), 4096, small[2].data_ptr(), 1, 1024, 24, 1024, 4096, None, stream) == 0, err().decode()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(DEV)[0] == free_before, "the entry point took or returned device memory"
    for out in outs:
        torch.testing.assert_close(out.float(), ref, rtol=1.6e-2, atol=2e-3)


def test_static_scratch_entry_refuses_a_plan_larger_than_its_array():
    """1,536 x 1,536 x 4,096: 36 tiles of 256 x 256, K in two ranges, 2 x 1,536 x 1,536 floats of
    partial products: more than the array's 4 Mi.  The call returns 1 with a message that gives
    both numbers, launches nothing (the output keeps what it held) and allocates nothing."""
    from spyinfer_b200.csrc import build
    fn, err = static_entry()
    M, N, K = 1536, 1536, 4096
    plan = build.load("gemm_tcgen05").spy_gemm_tcgen05_plan
    splits, need = ctypes.c_int(), ctypes.c_longlong()
    plan(M, N, K, ctypes.c_longlong(1 << 40), ctypes.byref(splits), ctypes.byref(need))
    assert splits.value == 2 and need.value == 2 * M * N > 4 * 1024 * 1024
    a = torch.zeros(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
    out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(DEV)[0]
    rc = fn(a.data_ptr(), K, w.data_ptr(), K, out.data_ptr(), 1, N, M, N, K, None, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 1
    message = err().decode()
    assert str(need.value) in message and str(4 * 1024 * 1024) in message, message
    assert torch.cuda.mem_get_info(DEV)[0] == free_before
    assert (out == 7.0).all()
