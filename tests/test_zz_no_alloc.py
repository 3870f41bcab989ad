"""The INT4 GEMV entry point that allocates nothing (scratch in a fixed array inside the library).

For callers that cannot provide a workspace because they must not allocate device memory - all of it belongs
to the application's own pool, or the call sits in a loop where cudaMalloc is ruled out.  The check: called
through the C ABI, it gives the same answer as the regular entry point (which takes a caller workspace), twice
in a row on the shared scratch.  Collected last on purpose, so that a run that stops at the first failure has
already exercised everything else.
"""
import numpy as np
import pytest
import torch

from helpers import awq_random, rel_err

pytestmark = pytest.mark.gpu


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


@pytest.mark.parametrize("M,K,N,residual", [(1, 4096, 4096, True), (3, 1024, 3072, False), (1, 256, 1056, True),
                                            (8, 256, 32768, False)])  # last: both limits at once (8 rows, widest N)
def test_noalloc_entry_matches_workspace_entry(cuda, oracle, M, K, N, residual):
    from mykuiperllama_b200._lib import check, kernels
    lib = kernels()
    assert lib.kuiper_awq_gemv_noalloc_scratch_bytes() == 256 + (512 + 32) * 1024 * 4
    rng = np.random.default_rng(K * 3 + N + M)
    q, z, s = awq_random(rng, K, N)
    qw, qz = _dev(oracle.awq_pack(q)), _dev(oracle.awq_pack(z))
    sc = _dev(s.view(np.uint16), torch.float16)
    x = _dev(rng.standard_normal((M, K)).astype(np.float32))
    res = _dev(rng.standard_normal((M, N)).astype(np.float32)) if residual else None
    want = cuda.awq_gemv(x, qw, qz, sc, residual=res).cpu().numpy()  # existing entry point, caller workspace
    # the checker's answer for the same inputs (activation rounded to fp16 as the kernel does)
    ref = oracle.awq_gemv(x.cpu().numpy(), oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16), acc_double=True,
                          act_round=oracle.ROUND_FP16).astype(np.float64)
    if residual:
        ref = ref + res.cpu().numpy()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    ys = [torch.full((M, N), float("nan"), device="cuda") for _ in range(2)]
    free_before = None
    for i in range(2):  # the second call finds the scratch as the first one left it
        y = ys[i]
        if i == 1:
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        check(lib.kuiper_awq_gemv_f32_noalloc(x.data_ptr(), qw.data_ptr(), qz.data_ptr(), sc.data_ptr(), y.data_ptr(),
                                              res.data_ptr() if residual else None, M, K, N, 128, stream))
        torch.cuda.synchronize()
        if i == 1:
            # the defining property: the device's free memory is the same before and after the call
            assert torch.cuda.mem_get_info()[0] == free_before
        outs.append(y.cpu().numpy())
    for y in outs:
        # same kernel, possibly a different grid: only the order of the fp32 partial sums may differ
        assert rel_err(y, want) <= 2e-6
        assert rel_err(y, ref) <= 2e-6
    assert np.array_equal(outs[0], outs[1])


def test_noalloc_entry_rejects_sizes_beyond_its_scratch(cuda):
    from mykuiperllama_b200._lib import kernels
    lib = kernels()
    one = torch.zeros(64, device="cuda")
    args = (one.data_ptr(),) * 5
    assert lib.kuiper_awq_gemv_f32_noalloc(*args, None, 1, 128, 32768 + 32, 128, None) == 7   # wider than the scratch
    assert b"exceeds" in lib.kuiper_last_error()
    assert lib.kuiper_awq_gemv_f32_noalloc(*args, None, 9, 128, 1024, 128, None) == 7         # more than 8 rows
    assert lib.kuiper_awq_gemv_f32_noalloc(*args, None, 1, 128, 1000, 128, None) == 7         # N % 32 != 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_noalloc_entry_on_a_second_device(cuda, oracle):
    # the scratch address, the shared-memory attribute of the kernel and the SM count are kept per device: a call on
    # device 1 after device 0 has been used must configure device 1 on its own
    from mykuiperllama_b200._lib import check, kernels
    lib = kernels()
    rng = np.random.default_rng(77)
    M, K, N = 2, 1024, 4096
    q, z, s = awq_random(rng, K, N)
    xh = rng.standard_normal((M, K)).astype(np.float32)
    ref = oracle.awq_gemv(xh, oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16), acc_double=True,
                          act_round=oracle.ROUND_FP16).astype(np.float64)
    for device in (0, 1, 0):
        with torch.cuda.device(device):
            dev = f"cuda:{device}"
            qw = torch.from_numpy(oracle.awq_pack(q)).to(dev)
            qz = torch.from_numpy(oracle.awq_pack(z)).to(dev)
            sc = torch.from_numpy(s.view(np.uint16).copy()).to(dev).view(torch.float16)
            x = torch.from_numpy(xh).to(dev)
            y = torch.full((M, N), float("nan"), device=dev)
            stream = torch.cuda.current_stream().cuda_stream
            check(lib.kuiper_awq_gemv_f32_noalloc(x.data_ptr(), qw.data_ptr(), qz.data_ptr(), sc.data_ptr(), y.data_ptr(),
                                                  None, M, K, N, 128, stream))
            torch.cuda.synchronize()
            assert rel_err(y.cpu().numpy(), ref) <= 2e-6, device
