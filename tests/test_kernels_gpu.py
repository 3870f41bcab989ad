"""Parity of every CUDA kernel (called through the C ABI) against the CPU oracle.

Tolerances: integer / byte results bit-exact; floating-point outputs within
max|y-ref|/max|ref| <= 1e-2 (the workload's stated bound), with a tighter engineering
bound asserted next to it so that a regression inside the allowed band is still seen.
"""
import numpy as np
import pytest
import torch

from helpers import awq_random, rel_err

pytestmark = pytest.mark.gpu

SPEC_TOL = 1e-2
GEMM_IMPL_DEFAULT = 3


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


# ----------------------------------------------------------------------------- add
@pytest.mark.parametrize("shape,a,b,expect,tol", [((32, 151), 2.0, 3.0, 5.0, 0.0), ((32, 151, 13), 2.1, 3.3, 5.4, 1e-4)])
def test_add_matches_reference_pins(cuda, shape, a, b, expect, tol):
    # the reference's own known answers: test/test_op/test_op_add.cpp:7-26 and :72-91
    x = torch.full(shape, a, device="cuda")
    y = torch.full(shape, b, device="cuda")
    out = cuda.add(x, y)
    torch.cuda.synchronize()
    assert float((out - expect).abs().max()) <= tol


def test_add_on_user_stream_and_unaligned(cuda, oracle):
    rng = np.random.default_rng(1)
    a = rng.standard_normal(4099).astype(np.float32)
    b = rng.standard_normal(4099).astype(np.float32)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):  # test_op_add.cpp:28-51 runs the kernel on a user stream
        ta, tb = dev(a), dev(b)
        out = cuda.add(ta[1:], tb[1:].clone())  # first operand 4-byte aligned only: scalar path
    s.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.add(a[1:], b[1:]))


# ----------------------------------------------------------------------------- AWQ unpack / dequant
def test_awq_unpack_and_dequant_bit_exact_c1(cuda, oracle):
    rng = np.random.default_rng(0)
    K = N = 2048
    q, z, s = awq_random(rng, K, N)
    qw, qz = oracle.awq_pack(q), oracle.awq_pack(z)
    su = s.view(np.uint16)
    got_q = cuda.awq_unpack(dev(qw)).cpu().numpy()
    assert np.array_equal(got_q, q)
    W_ref = oracle.awq_dequant(qw, qz, su)
    W = cuda.awq_dequant(dev(qw), dev(qz), dev(su)).cpu().numpy()
    assert np.array_equal(W.view(np.uint32), W_ref.view(np.uint32))
    Wb = cuda.awq_dequant(dev(qw), dev(qz), dev(su), dtype=torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(Wb, oracle.f32_to_bf16(W_ref))


# ----------------------------------------------------------------------------- AWQ GEMV
def _gemv_case(cuda, oracle, rng, M, K, N, act_mode, residual=False, rows=0):
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    x = rng.standard_normal((M, K)).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32) if residual else None
    ref = oracle.awq_gemv(x, qw, qz, su, acc_double=True)
    if residual:
        ref = (ref.astype(np.float64) + res).astype(np.float32)
    cuda.set_tuning("gemv_rows", rows)
    try:
        ws = cuda.awq_gemv_workspace(M, K, N)
        args = (dev(x), dev(qw), dev(qz), dev(su, torch.float16))
        y1 = cuda.awq_gemv(*args, workspace=ws, residual=dev(res) if residual else None, act_mode=act_mode)
        # second call on the same workspace: the arrival counters must have been left at zero
        y2 = cuda.awq_gemv(*args, workspace=ws, residual=dev(res) if residual else None, act_mode=act_mode)
        torch.cuda.synchronize()
    finally:
        cuda.set_tuning("gemv_rows", 0)
    y1, y2 = y1.cpu().numpy(), y2.cpu().numpy()
    assert np.array_equal(y1, y2), "split-K result depends on scheduling or stale counters"
    return rel_err(y1, ref), y1, ref, (x, qw, qz, su)


@pytest.mark.parametrize("act_mode,tight", [(1, 1e-3), (0, 2e-6)])
def test_awq_gemv_c1(cuda, oracle, act_mode, tight):
    # config 1 of the workload: x [1,2048] ~N(0,1), W 2048x2048, group 128, seed 0
    err, *_ = _gemv_case(cuda, oracle, np.random.default_rng(0), 1, 2048, 2048, act_mode)
    assert err <= SPEC_TOL
    assert err <= tight


def test_awq_gemv_fp16_mode_matches_mirrored_oracle(cuda, oracle):
    # the fp16 tensor-core kernel: with the activation rounded to fp16 in the oracle too, only the summation order differs
    for M in (1, 2):
        err, y, _, (x, qw, qz, su) = _gemv_case(cuda, oracle, np.random.default_rng(3), M, 4096, 1024, 1)
        ref16 = oracle.awq_gemv(x, qw, qz, su, acc_double=True, act_round=oracle.ROUND_FP16)
        assert rel_err(y, ref16) <= 2e-6


@pytest.mark.parametrize("M,K,N", [(1, 1024, 4096), (1, 4096, 6144), (1, 2560, 2560), (2, 1024, 3072), (3, 3072, 1024),
                                   (5, 512, 2048), (8, 256, 1056), (1, 128, 32), (1, 12288, 4096)])
@pytest.mark.parametrize("rows", [0, 4, 8, 16])
def test_awq_gemv_shapes(cuda, oracle, M, K, N, rows):
    if rows and K % (rows * 8):
        pytest.skip("K slice does not divide K")
    err, *_ = _gemv_case(cuda, oracle, np.random.default_rng(M * 7 + K + N), M, K, N, 1, residual=(M % 2 == 1), rows=rows)
    assert err <= 1e-3


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 4096, 6144), (1, 12288, 4096), (2, 1024, 3072), (3, 256, 1056), (1, 128, 32),
                                   (1, 2560, 2560)])
def test_awq_gemv_accumulate_mode(cuda, oracle, M, K, N):
    # y += x.W on top of an addend already in y (the engine's path: residual stream or zeros)
    rng = np.random.default_rng(K + N + M)
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    x = rng.standard_normal((M, K)).astype(np.float32)
    addend = rng.standard_normal((M, N)).astype(np.float32)
    ref = oracle.awq_gemv(x, qw, qz, su, act_round=oracle.ROUND_FP16).astype(np.float64) + addend
    y = dev(addend)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        cuda.awq_gemv_accum(dev(x), dev(qw), dev(qz), dev(su, torch.float16), y)
    side.synchronize()
    err = rel_err(y.cpu().numpy(), ref)
    assert err <= SPEC_TOL and err <= 2e-6  # only the (unordered) fp32 summation differs from the mirrored oracle
    cuda.awq_gemv_status()


@pytest.mark.parametrize("M,K,N", [(1, 4096, 6144), (2, 1024, 2048), (1, 2560, 1056), (3, 256, 1024)])
def test_rmsnorm_fused_into_accumulating_gemv(cuda, oracle, M, K, N):
    rng = np.random.default_rng(K * 5 + N + M)
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    h = (rng.standard_normal((M, K)) * 2.5).astype(np.float32)
    nw = oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(K)).astype(np.float32))
    addend = rng.standard_normal((M, N)).astype(np.float32)
    xn = oracle.rmsnorm(h, nw, 1e-6)
    ref = oracle.awq_gemv(xn, qw, qz, su).astype(np.float64) + addend  # un-rounded operand: the workload's reference
    y = dev(addend)
    cuda.rmsnorm_awq_gemv_accum(dev(h), dev(nw), 1e-6, dev(qw), dev(qz), dev(su, torch.float16), y)
    torch.cuda.synchronize()
    err = rel_err(y.cpu().numpy(), ref)
    assert err <= SPEC_TOL and err <= 1e-3


@pytest.mark.parametrize("M,K,N", [(1, 12288, 4096), (2, 1024, 2048), (4, 3072, 1024), (1, 256, 1056)])
def test_swiglu_fused_into_accumulating_gemv(cuda, oracle, M, K, N):
    # y += (silu(gate) * up) . W: the activation is formed by the kernel's activation warp, gate|up is only read
    rng = np.random.default_rng(M + K + N)
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    gu = rng.standard_normal((M, 2 * K)).astype(np.float32)
    addend = rng.standard_normal((M, N)).astype(np.float32)
    act = np.stack([oracle.swiglu(gu[m, :K], gu[m, K:]) for m in range(M)])
    ref = oracle.awq_gemv(act, qw, qz, su, act_round=oracle.ROUND_FP16).astype(np.float64) + addend
    y, tgu = dev(addend), dev(gu)
    cuda.swiglu_awq_gemv_accum(tgu, dev(qw), dev(qz), dev(su, torch.float16), y)
    torch.cuda.synchronize()
    err = rel_err(y.cpu().numpy(), ref)
    assert err <= SPEC_TOL and err <= 1e-5  # expf may differ by an ulp between host and device
    assert np.array_equal(tgu.cpu().numpy(), gu)
    cuda.awq_gemv_status()


@pytest.mark.parametrize("K,N", [(4096, 24576), (2560, 19456), (9728, 2560), (2560, 6144)])
def test_awq_gemv_layer_shapes_of_the_4b_and_8b_models_match_oracle(cuda, oracle, K, N):
    # the widest projection of the 8B shape and the three distinct 4B shapes, against the oracle (not a property test):
    # accumulate entry, fused-RMSNorm entry and - with K as the SwiGLU width - the fused-SwiGLU entry
    rng = np.random.default_rng(K * 7 + N)
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    W = (dev(qw), dev(qz), dev(su, torch.float16))
    addend = rng.standard_normal((1, N)).astype(np.float32)
    x = rng.standard_normal((1, K)).astype(np.float32)
    y = dev(addend)
    cuda.awq_gemv_accum(dev(x), *W, y)
    ref = oracle.awq_gemv(x, qw, qz, su, acc_double=True)
    err = rel_err(y.cpu().numpy(), ref.astype(np.float64) + addend)
    assert err <= SPEC_TOL and err <= 1e-3                      # against the un-rounded oracle: the workload's bound
    ref16 = oracle.awq_gemv(x, qw, qz, su, acc_double=True, act_round=oracle.ROUND_FP16)
    assert rel_err(y.cpu().numpy(), ref16.astype(np.float64) + addend) <= 2e-6   # mirrored operand rounding
    # ordered-combine entry (deterministic summation order) on the same matrix
    yo = cuda.awq_gemv(dev(x), *W, residual=dev(addend))
    assert rel_err(yo.cpu().numpy(), ref16.astype(np.float64) + addend) <= 2e-6
    nw = oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(K)).astype(np.float32))
    h = (x * 2.5).astype(np.float32)
    y = dev(addend)
    cuda.rmsnorm_awq_gemv_accum(dev(h), dev(nw), 1e-6, *W, y)
    ref = oracle.awq_gemv(oracle.rmsnorm(h, nw, 1e-6), qw, qz, su, acc_double=True).astype(np.float64) + addend
    err = rel_err(y.cpu().numpy(), ref)
    assert err <= SPEC_TOL and err <= 1e-3
    gu = rng.standard_normal((1, 2 * K)).astype(np.float32)
    y = dev(addend)
    cuda.swiglu_awq_gemv_accum(dev(gu), *W, y)
    act = oracle.swiglu(gu[0, :K], gu[0, K:])[None, :]
    ref = oracle.awq_gemv(act, qw, qz, su, acc_double=True, act_round=oracle.ROUND_FP16).astype(np.float64) + addend
    err = rel_err(y.cpu().numpy(), ref)
    assert err <= SPEC_TOL and err <= 1e-5
    cuda.awq_gemv_status()


@pytest.mark.parametrize("M,K,N,kind", [(1, 4096, 6144, "norm"), (1, 12288, 4096, "swiglu"), (1, 4096, 24576, "plain"), (2, 1024, 3072, "plain"),
                                        (4, 2560, 1056, "norm"), (1, 128, 32, "plain"), (1, 4096, 4096, "plain")])
@pytest.mark.parametrize("pct,chunk", [(25, 0), (90, 1), (50, 3)])
@pytest.mark.parametrize("act_mode", [1, 2])
def test_awq_gemv_balanced_by_tickets_matches_oracle(cuda, oracle, M, K, N, kind, pct, chunk, act_mode):
    # the engine's entry: a share of the weight stream is handed out through an atomic ticket counter; whatever CTA
    # takes which unit, the sum is the oracle's, and the counters are back at zero after every launch
    rng = np.random.default_rng(M + K + N + pct)
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    W = (dev(qw), dev(qz), dev(su, torch.float16))
    addend = rng.standard_normal((M, N)).astype(np.float32)
    tickets = cuda.awq_gemv_tickets()
    cuda.set_tuning("gemv_dyn_pct", pct)
    cuda.set_tuning("gemv_dyn_chunk", chunk)
    # act_mode 2: a one-row call rounds its operand to 16-bit block floating point (integer tensor-core kernel), calls
    # with more rows to fp16 - the oracle's ROUND_ENGINE does the same
    mirror = oracle.ROUND_ENGINE if act_mode == 2 else oracle.ROUND_FP16
    try:
        for rep in range(3):  # the second and third launch find the counters as the one before left them
            y = dev(addend)
            if kind == "norm":
                h = (rng.standard_normal((M, K)) * 2.5).astype(np.float32)
                nw = oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(K)).astype(np.float32))
                cuda.awq_gemv_accum_balanced(dev(h), *W, y, tickets, norm_w=dev(nw), eps=1e-6, act_mode=act_mode)
                ref, tol = oracle.awq_gemv(oracle.rmsnorm(h, nw, 1e-6), qw, qz, su).astype(np.float64) + addend, 1e-3
            elif kind == "swiglu":
                gu = rng.standard_normal((M, 2 * K)).astype(np.float32)
                cuda.awq_gemv_accum_balanced(dev(gu), *W, y, tickets, swiglu=True, act_mode=act_mode)
                act = np.stack([oracle.swiglu(gu[m, :K], gu[m, K:]) for m in range(M)])
                ref, tol = oracle.awq_gemv(act, qw, qz, su, act_round=mirror).astype(np.float64) + addend, 1e-5
            else:
                x = rng.standard_normal((M, K)).astype(np.float32)
                cuda.awq_gemv_accum_balanced(dev(x), *W, y, tickets, act_mode=act_mode)
                ref, tol = oracle.awq_gemv(x, qw, qz, su, act_round=mirror).astype(np.float64) + addend, 2e-6
            torch.cuda.synchronize()
            err = rel_err(y.cpu().numpy(), ref)
            assert err <= SPEC_TOL and err <= tol, (rep, err)
            assert not tickets.any(), "the ticket and exit counters must be back at zero after the launch"
    finally:
        cuda.set_tuning("gemv_dyn_pct", -1)
        cuda.set_tuning("gemv_dyn_chunk", -1)
    cuda.awq_gemv_status()


@pytest.mark.parametrize("shapes", [[(2048, 2048)] * 9, [(256, 1056), (4096, 4096), (128, 32), (1024, 3072), (2560, 2560)],
                                    [(128, 32)] * 3, [(2048, 2048)] * 70])
@pytest.mark.parametrize("balanced,act_mode", [(True, 1), (False, 1), (False, 2), (True, 2)])
def test_awq_gemv_grouped_launch_matches_oracle(cuda, oracle, shapes, balanced, act_mode):
    # a list of independent projections as ONE persistent launch (the single-GEMV workload visited over many weight
    # sets): every item against the oracle, twice on the same table and counters
    rng = np.random.default_rng(len(shapes) * 13 + shapes[0][0])
    items, refs = [], []
    distinct = {}
    for i, (K, N) in enumerate(shapes):
        key = (K, N, i % 5)  # a handful of distinct weight sets per shape keeps the oracle's share of the test short
        if key not in distinct:
            q, z, s = awq_random(rng, K, N)
            distinct[key] = (oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16))
        qw, qz, su = distinct[key]
        x = rng.standard_normal((1, K)).astype(np.float32)
        addend = rng.standard_normal((1, N)).astype(np.float32)
        items.append(dict(x=dev(x), qweight=dev(qw), qzeros=dev(qz), scales=dev(su, torch.float16), y=dev(addend)))
        refs.append((oracle.awq_gemv(x, qw, qz, su, act_round=oracle.ROUND_FP16 if act_mode == 1 else oracle.ROUND_I16_BLOCK32).astype(np.float64),
                     addend))
    grp = cuda.GemvGroup(items, balanced=balanced, act_mode=act_mode)
    for rep in (1, 2):
        grp.run()
        torch.cuda.synchronize()
        for it, (ref, addend) in zip(items, refs):
            assert rel_err(it["y"].cpu().numpy(), rep * ref + addend) <= 4e-6
        if balanced:
            assert not grp.tickets.any()
    cuda.awq_gemv_status()


@pytest.mark.parametrize("K,N", [(4096, 4096), (2048, 2048), (256, 1056), (128, 32), (12288, 4096)])
@pytest.mark.parametrize("scale", [1.0, 1e-6, 3e4])
def test_awq_gemv_integer_operand_kernel(cuda, oracle, K, N, scale):
    # one token row on the integer tensor path (act_mode 2): the operand is 16-bit block floating point per 32 rows, every
    # product and every sum inside a block is an exact integer.  Against the oracle with the same operand rounding only
    # the fp32 summation across blocks differs; against the un-rounded oracle the workload's 1e-2 holds with a wide
    # margin also when the activations are tiny, large, or carry outliers
    rng = np.random.default_rng(K + N)
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    W = (dev(qw), dev(qz), dev(su, torch.float16))
    x = (rng.standard_normal((1, K)) * scale).astype(np.float32)
    x[0, ::97] *= 300.0  # outliers inside many blocks
    res = (rng.standard_normal((1, N)) * scale).astype(np.float32)
    ref_mirror = oracle.awq_gemv(x, qw, qz, su, acc_double=True, act_round=oracle.ROUND_I16_BLOCK32).astype(np.float64) + res
    ref_plain = oracle.awq_gemv(x, qw, qz, su, acc_double=True).astype(np.float64) + res
    y = cuda.awq_gemv(dev(x), *W, residual=dev(res), act_mode=2)          # ordered combine: deterministic
    y2 = cuda.awq_gemv(dev(x), *W, residual=dev(res), act_mode=2)
    ya = dev(res)
    cuda.awq_gemv_accum_balanced(dev(x), *W, ya, act_mode=2)               # accumulate mode
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    for got in (y.cpu().numpy(), ya.cpu().numpy()):
        assert rel_err(got, ref_mirror) <= 2e-6
        err = rel_err(got, ref_plain)
        assert err <= SPEC_TOL and err <= 1e-3
    cuda.awq_gemv_status()


def test_awq_gemv_ragged_width_uses_generic_kernel(cuda, oracle):
    err, *_ = _gemv_case(cuda, oracle, np.random.default_rng(5), 2, 256, 40, 1, residual=True)
    assert err <= 2e-6


def test_awq_gemv_half2_mode_within_spec(cuda, oracle):
    cuda.set_tuning("gemv_math", 2)
    try:
        err, *_ = _gemv_case(cuda, oracle, np.random.default_rng(0), 1, 2048, 2048, 1)
    finally:
        cuda.set_tuning("gemv_math", -1)
    assert err <= SPEC_TOL


def test_awq_gemv_linearity_full_size(cuda, oracle):
    # size-independent property at the largest layer shape: W(a*x1 + x2) == a*W(x1) + W(x2)
    rng = np.random.default_rng(11)
    K, N = 4096, 24576
    qw = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int32, device="cuda")
    qz = torch.randint(-2**31, 2**31 - 1, (K // 128, N // 8), dtype=torch.int32, device="cuda")
    s = (torch.rand((K // 128, N), device="cuda") * 0.018 + 0.002).half()
    x1, x2 = dev(rng.standard_normal((1, K)).astype(np.float32)), dev(rng.standard_normal((1, K)).astype(np.float32))
    ws = cuda.awq_gemv_workspace(1, K, N)
    f = lambda x: cuda.awq_gemv(x, qw, qz, s, workspace=ws, act_mode=0)
    lhs = f(0.5 * x1 + x2)
    rhs = 0.5 * f(x1) + f(x2)
    torch.cuda.synchronize()
    assert rel_err(lhs.cpu().numpy(), rhs.cpu().numpy()) <= 1e-5


def test_awq_gemv_rejects_bad_arguments(cuda):
    from mykuiperllama_b200._lib import KuiperError
    x = torch.zeros((1, 192), device="cuda")
    qw = torch.zeros((192, 4), dtype=torch.int32, device="cuda")
    qz = torch.zeros((2, 4), dtype=torch.int32, device="cuda")
    s = torch.zeros((2, 32), dtype=torch.float16, device="cuda")
    with pytest.raises(KuiperError) as e:  # K not a multiple of the group
        cuda.awq_gemv(x, qw, qz, s)
    assert e.value.code == 7
    with pytest.raises(KuiperError) as e:  # unsupported group
        cuda.awq_gemv(torch.zeros((1, 256), device="cuda"), torch.zeros((256, 4), dtype=torch.int32, device="cuda"), qz, s, group=64)
    assert e.value.code == 7


# ----------------------------------------------------------------------------- INT4 GEMM (tcgen05), M >= 16
@pytest.mark.parametrize("M,K,N", [(16, 128, 128), (16, 256, 136), (100, 1024, 384), (128, 4096, 1024), (129, 512, 256),
                                   (300, 1024, 4104), (16, 4096, 6144), (64, 3072, 1024)])
@pytest.mark.parametrize("impl,split_k", [(3, 1), (3, 0), (2, 0)])  # 3: mbarrier hand-over to a dedicated MMA warp, with
def test_awq_gemm_tensor_core(cuda, oracle, M, K, N, impl, split_k):     # and without the K split; 2: block-wide barrier
    cuda.set_tuning("gemm_impl", impl)
    cuda.set_tuning("gemm_split_k", split_k)
    try:
        _gemm_case(cuda, oracle, M, K, N, exact=not split_k)
    finally:
        cuda.set_tuning("gemm_impl", GEMM_IMPL_DEFAULT)
        cuda.set_tuning("gemm_split_k", 1)


def _gemm_case(cuda, oracle, M, K, N, exact):
    rng = np.random.default_rng(M + K + N)
    q, z, s = awq_random(rng, K, N)
    qw, qz, su = oracle.awq_pack(q), oracle.awq_pack(z), s.view(np.uint16)
    x = rng.standard_normal((M, K)).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    ref = oracle.awq_gemv(x, qw, qz, su, act_round=oracle.ROUND_FP16).astype(np.float64)
    tx, tqw, tqz, ts = dev(x), dev(qw), dev(qz), dev(su, torch.float16)
    ws = cuda.awq_gemm_workspace(M, K)
    y = cuda.awq_gemm(tx, tqw, tqz, ts, workspace=ws)
    y_res = cuda.awq_gemm(tx, tqw, tqz, ts, residual=dev(res), workspace=ws)
    y_acc = dev(res)
    cuda.awq_gemm(tx, tqw, tqz, ts, y=y_acc, accumulate=True, workspace=ws)
    torch.cuda.synchronize()
    # the weight (q - z) * s is rounded to fp16 before the tensor-core product: ~2^-11 per weight on top of the GEMV's error
    err = rel_err(y.cpu().numpy(), ref)
    assert err <= SPEC_TOL and err <= 1e-3
    assert rel_err(y_res.cpu().numpy(), ref + res) <= 1e-3
    again = cuda.awq_gemm(tx, tqw, tqz, ts, workspace=ws)
    torch.cuda.synchronize()
    if exact:
        assert torch.equal(y_acc, y_res)  # same tile, same order: bit-identical
        assert torch.equal(again, y)      # fixed summation order: deterministic
    else:  # the K split adds its partial sums with reductions: only the fp32 summation order may differ
        assert rel_err(y_acc.cpu().numpy(), y_res.cpu().numpy()) <= 2e-6
        assert rel_err(again.cpu().numpy(), y.cpu().numpy()) <= 2e-6
    cuda.awq_gemm_status()


def test_awq_gemm_agrees_with_gemv_rows(cuda, oracle):
    # the batched-decode switch (M >= 16 -> GEMM) must not move results beyond the fp16 weight rounding
    rng = np.random.default_rng(77)
    M, K, N = 16, 1024, 2048
    q, z, s = awq_random(rng, K, N)
    tqw, tqz, ts = dev(oracle.awq_pack(q)), dev(oracle.awq_pack(z)), dev(s.view(np.uint16), torch.float16)
    x = dev(rng.standard_normal((M, K)).astype(np.float32))
    y = cuda.awq_gemm(x, tqw, tqz, ts)
    rows = torch.cat([cuda.awq_gemv(x[i:i + 8].contiguous(), tqw, tqz, ts) for i in range(0, M, 8)])
    torch.cuda.synchronize()
    assert rel_err(y.cpu().numpy(), rows.cpu().numpy()) <= 1e-3


def test_awq_gemm_rejects_bad_arguments(cuda):
    from mykuiperllama_b200._lib import KuiperError
    qz = torch.zeros((2, 4), dtype=torch.int32, device="cuda")
    s = torch.zeros((2, 32), dtype=torch.float16, device="cuda")
    with pytest.raises(KuiperError) as e:  # K not a multiple of the group
        cuda.awq_gemm(torch.zeros((16, 192), device="cuda"), torch.zeros((192, 4), dtype=torch.int32, device="cuda"), qz, s)
    assert e.value.code == 7
    x = torch.zeros((16, 256), device="cuda")
    qw = torch.zeros((256, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(KuiperError) as e:  # accumulate and residual at once
        cuda.awq_gemm(x, qw, qz, s, y=torch.zeros((16, 32), device="cuda"), residual=torch.zeros((16, 32), device="cuda"),
                      accumulate=True)
    assert e.value.code == 7


# ----------------------------------------------------------------------------- tensor-parallel exchanges (single-GPU checks)
def _words(values, seq):
    """8-byte exchange words {value bits, sequence number} as an int32 tensor [n, 2]."""
    v = np.ascontiguousarray(values)
    w = np.empty((v.size, 2), np.uint32)
    w[:, 0] = v.view(np.uint32).ravel()
    w[:, 1] = seq
    return torch.from_numpy(w.view(np.int32)).cuda()


def test_allreduce_sum_two_ranks_emulated_on_one_gpu(cuda, oracle):
    # Both "ranks" live on this GPU and their kernels would run one after the other on one stream, so rank 0 could never
    # see rank 1's words: rank 1's slot in rank 0's buffer is filled by hand instead, then rank 0 runs alone.
    rng = np.random.default_rng(41)
    world, count, max_count = 2, 4096, 8192
    bufs = [cuda.allreduce_buffer(world, max_count) for _ in range(world)]
    state = cuda.allreduce_state()
    a = rng.standard_normal(count).astype(np.float32)
    b = rng.standard_normal(count).astype(np.float32)
    h = rng.standard_normal(count).astype(np.float32)
    # sequence number 1 -> parity 1; sum slot (parity 1, src 1) of rank 0's buffer
    words = bufs[0].view(torch.int32).view(-1, 2)
    slot = (1 * world + 1) * max_count
    words[slot:slot + count] = _words(b, 1)
    partial, resid = dev(a), dev(h)
    out = cuda.allreduce_sum(partial, 0, world, bufs, max_count, state, residual=resid, clear_partial=True)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), (h + a) + b)  # residual first, then the ranks in order
    assert float(partial.abs().max()) == 0.0               # cleared for the next accumulating projection
    st = state.cpu().numpy()
    assert list(st[:4]) == [1, 1, 1, 1] and st[64 + 1] == 0  # four CTAs advanced their sequence numbers, no error
    # rank 0 also delivered its words to "rank 1": slot (parity 1, src 0) of rank 1's buffer
    got = bufs[1].view(torch.int32).view(-1, 2)[(1 * world + 0) * max_count:(1 * world + 0) * max_count + count].cpu().numpy()
    assert np.array_equal(got[:, 0].view(np.float32), a) and (got[:, 1] == 1).all()
    cuda.allreduce_status(state)


def test_argmax_allgather_two_ranks_emulated_on_one_gpu(cuda, oracle):
    rng = np.random.default_rng(43)
    world, M, V_local, max_count = 2, 3, 18992, 8192
    bufs = [cuda.allreduce_buffer(world, max_count) for _ in range(world)]
    state = cuda.allreduce_state()
    full = rng.standard_normal((M, world * V_local)).astype(np.float32)
    full[1, 77] = full[1, V_local + 5] = 9.0   # tie across the two slices: the lower global index wins
    full[2, V_local + 18991] = 50.0            # last element of the upper slice
    want = oracle.argmax(full)
    # rank 1's (maximum, index) words, by hand, into rank 0's buffer: argmax slot (parity 1, src 1)
    hi = full[:, V_local:]
    idx1 = hi.argmax(1)
    base = 2 * world * max_count * 8 + (1 * world + 1) * 16 * 16
    area = bufs[0][base:base + M * 16].view(torch.int32).view(M, 2, 2)
    area[:, 0] = _words(hi[np.arange(M), idx1], 1)
    area[:, 1] = _words((idx1 + V_local).astype(np.uint32).view(np.float32), 1)
    got = cuda.argmax_allgather(dev(np.ascontiguousarray(full[:, :V_local])), 0, world, bufs, max_count, state)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), want)
    assert got.cpu().tolist()[1] == 77
    cuda.allreduce_status(state)


def test_exchange_waits_are_bounded(cuda):
    # a peer whose words never arrive: the kernels give up after the time limit, report which rank, and the context
    # stays usable; the error word can be cleared
    from mykuiperllama_b200._lib import KuiperError
    world, count, max_count = 2, 1024, 1024
    bufs = [cuda.allreduce_buffer(world, max_count) for _ in range(world)]
    state = cuda.allreduce_state()
    cuda.set_tuning("allreduce_timeout_ms", 50)
    try:
        cuda.allreduce_sum(torch.ones(count, device="cuda"), 0, world, bufs, max_count, state)
        torch.cuda.synchronize()
        with pytest.raises(KuiperError) as e:
            cuda.allreduce_status(state, clear=True)
        assert e.value.code == 5 and "rank 1" in str(e.value)
        cuda.allreduce_status(state)  # cleared
        assert state.cpu().tolist()[0] == 1  # the sequence number still advanced
        cuda.argmax_allgather(torch.zeros((2, 64), device="cuda"), 0, world, bufs, max_count, state)
        torch.cuda.synchronize()
        with pytest.raises(KuiperError) as e:
            cuda.allreduce_status(state)
        assert e.value.code == 5
    finally:
        cuda.set_tuning("allreduce_timeout_ms", 5000)
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


# ----------------------------------------------------------------------------- BF16 GEMV
@pytest.mark.parametrize("M,K,N", [(1, 1024, 5000), (1, 2560, 1001), (3, 4096, 2048), (4, 1024, 777), (7, 520, 64),
                                   (8, 2560, 3001), (16, 4096, 1000), (5, 1024, 9), (20, 1024, 100)])  # 3+ rows: tensor cores
def test_bf16_gemv(cuda, oracle, M, K, N):
    rng = np.random.default_rng(K + N)
    W = oracle.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((M, K)).astype(np.float32)
    ref = oracle.bf16_gemv(x, W)
    y = cuda.bf16_gemv(dev(x), dev(W)).cpu().numpy()
    err = rel_err(y, ref)
    assert err <= SPEC_TOL and err <= 2e-6


# ----------------------------------------------------------------------------- element-wise ops
@pytest.mark.parametrize("M,H", [(1, 1024), (3, 2560), (2, 4096), (1, 100)])
def test_rmsnorm(cuda, oracle, M, H):
    rng = np.random.default_rng(H)
    x = (rng.standard_normal((M, H)) * 3).astype(np.float32)
    w = oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(H)).astype(np.float32))
    y = cuda.rmsnorm(dev(x), dev(w), 1e-6).cpu().numpy()
    assert rel_err(y, oracle.rmsnorm(x, w, 1e-6)) <= 1e-6


def test_swiglu(cuda, oracle):
    rng = np.random.default_rng(2)
    gu = (rng.standard_normal((3, 2 * 3072)) * 4).astype(np.float32)
    ref = np.stack([oracle.swiglu(gu[m, :3072], gu[m, 3072:]) for m in range(3)])
    y = cuda.swiglu(dev(gu)).cpu().numpy()
    assert rel_err(y, ref) <= 1e-6


def test_swiglu_and_rope_can_clear_their_input(cuda, oracle):
    # the accumulating matmuls need their output buffer zero again after the consumer has read it
    rng = np.random.default_rng(12)
    gu = dev((rng.standard_normal((2, 2 * 512)) * 3).astype(np.float32))
    ref = cuda.swiglu(gu.clone()).cpu().numpy()
    out = cuda.swiglu(gu, clear_input=True)
    assert np.array_equal(out.cpu().numpy(), ref) and float(gu.abs().max()) == 0.0
    Nq, Nkv, D = 4, 2, 128
    qkv = dev(rng.standard_normal((3, (Nq + 2 * Nkv) * D)).astype(np.float32))
    qn = dev(oracle.f32_to_bf16(np.ones(D, np.float32)))
    cos_t, sin_t = oracle.rope_tables(16, D, 1e6)
    pos, slot = dev(np.array([0, 1, 2], np.int32)), dev(np.zeros(3, np.int32))
    kc = torch.zeros((1, Nkv, 16, D), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q1 = cuda.qknorm_rope_kvwrite(qkv.clone(), qn, qn, dev(cos_t), dev(sin_t), pos, slot, Nq, Nkv, D, 1e-6, kc.clone(), vc.clone())
    q2 = cuda.qknorm_rope_kvwrite(qkv, qn, qn, dev(cos_t), dev(sin_t), pos, slot, Nq, Nkv, D, 1e-6, kc, vc, clear_input=True)
    assert torch.equal(q1, q2) and float(qkv.abs().max()) == 0.0


def test_rope_kernel_clears_a_side_buffer(cuda, oracle):
    rng = np.random.default_rng(9)
    M, Nq, Nkv, D = 2, 4, 2, 128
    qkv = dev(rng.standard_normal((M, (Nq + 2 * Nkv) * D)).astype(np.float32))
    w = dev(oracle.f32_to_bf16(np.ones(D, np.float32)))
    cos_t, sin_t = (dev(t) for t in oracle.rope_tables(16, D, 1e6))
    kc = torch.zeros((1, Nkv, 16, D), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    side = torch.ones((M, 1000), device="cuda")
    keep = torch.ones(64, device="cuda")
    cuda.qknorm_rope_kvwrite(qkv, w, w, cos_t, sin_t, dev(np.array([3, 4], np.int32)), dev(np.zeros(2, np.int32)), Nq, Nkv, D,
                             1e-6, kc, vc, clear_input=True, clear_extra=side)
    torch.cuda.synchronize()
    assert float(side.abs().max()) == 0.0 and float(qkv.abs().max()) == 0.0 and float(keep.min()) == 1.0


def test_embedding_is_exact(cuda, oracle):
    rng = np.random.default_rng(4)
    table = oracle.f32_to_bf16(rng.standard_normal((1000, 1024)).astype(np.float32))
    tok = rng.integers(0, 1000, 9).astype(np.int32)
    y = cuda.embedding(dev(tok), dev(table)).cpu().numpy()
    assert np.array_equal(y, oracle.embedding(tok, table))


def test_argmax_lowest_index_on_ties(cuda, oracle):
    rng = np.random.default_rng(6)
    logits = rng.standard_normal((4, 151936)).astype(np.float32)
    logits[1, 77] = logits[1, 140000] = 9.0  # tie: lowest index wins
    logits[2, :] = 0.0                       # all equal: index 0
    logits[3, 151935] = 50.0                 # last element
    got = cuda.argmax(dev(logits)).cpu().numpy()
    assert np.array_equal(got, oracle.argmax(logits))
    assert got[1] == 77 and got[2] == 0 and got[3] == 151935


# ----------------------------------------------------------------------------- rotary + cache write
def test_qknorm_rope_kvwrite(cuda, oracle):
    rng = np.random.default_rng(8)
    M, Nq, Nkv, D, max_seq, slots = 5, 16, 8, 128, 64, 2
    qkv = rng.standard_normal((M, (Nq + 2 * Nkv) * D)).astype(np.float32)
    qn = oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32))
    kn = oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32))
    cos_t, sin_t = oracle.rope_tables(max_seq, D, 1e6)
    pos = np.array([0, 1, 17, 63, 5], np.int32)
    slot = np.array([0, 0, 1, 1, 1], np.int32)
    kc = np.zeros((slots, Nkv, max_seq, D), np.uint16)
    vc = np.zeros_like(kc)
    q_ref = oracle.qknorm_rope_kvwrite(qkv, qn, kn, cos_t, sin_t, pos, slot, Nq, Nkv, D, 1e-6, kc, vc)
    kc_d = torch.zeros((slots, Nkv, max_seq, D), dtype=torch.bfloat16, device="cuda")
    vc_d = torch.zeros_like(kc_d)
    q = cuda.qknorm_rope_kvwrite(dev(qkv), dev(qn), dev(kn), dev(cos_t), dev(sin_t), dev(pos), dev(slot),
                                 Nq, Nkv, D, 1e-6, kc_d, vc_d)
    torch.cuda.synchronize()
    assert rel_err(q.cpu().numpy(), q_ref) <= 1e-6
    # V is a pure bf16 rounding: bit-exact; K goes through a norm whose sum order differs: 1 bf16 ulp at most, rarely
    assert np.array_equal(vc_d.view(torch.int16).cpu().numpy().view(np.uint16), vc)
    k_got = oracle.bf16_to_f32(kc_d.view(torch.int16).cpu().numpy().view(np.uint16))
    k_ref = oracle.bf16_to_f32(kc)
    assert np.abs(k_got - k_ref).max() <= 2 ** -7 * np.abs(k_ref).max()
    assert (k_got != k_ref).mean() < 1e-3


# ----------------------------------------------------------------------------- flash decoding
FLASH_MMA_FUSED_DEFAULT = 1  # same for the fused rotary + attention kernel (key flash_mma_fused)
FLASH_MMA_DEFAULT = 1  # what the library starts with (kuiper_set_tuning key flash_mma)


@pytest.mark.parametrize("B,Nq,Nkv,lens", [
    (1, 32, 8, [1024]), (2, 32, 8, [4096, 777]), (1, 16, 8, [192]), (3, 8, 8, [1, 64, 65]),
    (4, 32, 8, [0, 63, 2048, 300]), (1, 32, 8, [16384]),
])
@pytest.mark.parametrize("splits", [0, 1, 7])
@pytest.mark.parametrize("tensor_cores", [0, 1])
def test_flash_decode(cuda, oracle, B, Nq, Nkv, lens, splits, tensor_cores):
    # tensor_cores = 1: the contractions run on mma.sync (bf16 cache rows as exact operands, q and the
    # probabilities as bf16 high + low parts); same grid, slices and combine
    rng = np.random.default_rng(sum(lens) + Nq + splits)
    D = 128
    max_seq = max(64, max(lens))
    q = rng.standard_normal((B, Nq, D)).astype(np.float32)
    kc = oracle.f32_to_bf16(rng.standard_normal((B, Nkv, max_seq, D)).astype(np.float32))
    vc = oracle.f32_to_bf16(rng.standard_normal((B, Nkv, max_seq, D)).astype(np.float32))
    seq = np.array(lens, np.int32)
    slot = np.arange(B, dtype=np.int32)[::-1].copy()  # rows read sequences in reverse order
    ref = oracle.attention(q, kc, vc, seq, slot)
    cuda.set_tuning("flash_splits", splits)
    cuda.set_tuning("flash_mma", tensor_cores)
    try:
        ws = cuda.flash_decode_workspace(B, Nq, D, max_seq)
        args = (dev(q), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), dev(seq), dev(slot))
        out1 = cuda.flash_decode(*args, workspace=ws).cpu().numpy()
        out2 = cuda.flash_decode(*args, workspace=ws).cpu().numpy()
    finally:
        cuda.set_tuning("flash_splits", 0)
        cuda.set_tuning("flash_mma", FLASH_MMA_DEFAULT)
    assert np.array_equal(out1, out2)
    err = rel_err(out1, ref)
    # 16 significant bits in q and in the probabilities on the tensor-core path
    assert err <= SPEC_TOL and err <= (5e-5 if tensor_cores else 1e-5)


_C3_CACHE = {}


def _c3_case(oracle, name):
    """Attention-workload extremes: batch 16 with mixed lengths (one at 32 768) and batch 1 at 32 768.  The caches are
    drawn on the GPU (N(0,1) rounded to bf16) and copied to the host for the oracle; the oracle's answer is kept for
    the second kernel."""
    if name in _C3_CACHE:
        return _C3_CACHE[name]
    lens = {"b16": [32768, 1, 64, 65, 4096, 777, 2048, 16384, 300, 1024, 5000, 63, 192, 8191, 12000, 31], "b1": [32768]}[name]
    B, Nq, Nkv, D, max_seq = len(lens), 32, 8, 128, 32768
    gen = torch.Generator(device="cuda")
    gen.manual_seed(321 + B)
    kc = torch.randn((B, Nkv, max_seq, D), device="cuda", generator=gen).bfloat16()
    vc = torch.randn((B, Nkv, max_seq, D), device="cuda", generator=gen).bfloat16()
    q = torch.randn((B, Nq, D), device="cuda", generator=gen)
    seq = np.array(lens, np.int32)
    slot = np.arange(B, dtype=np.int32)[::-1].copy()
    ref = oracle.attention(q.cpu().numpy(), kc.view(torch.int16).cpu().numpy().view(np.uint16),
                           vc.view(torch.int16).cpu().numpy().view(np.uint16), seq, slot)
    _C3_CACHE.clear()  # one case (up to 2 GB of cache) alive at a time
    _C3_CACHE[name] = (q, kc, vc, seq, slot, ref)
    return _C3_CACHE[name]


@pytest.mark.parametrize("name", ["b16", "b1"])
@pytest.mark.parametrize("tensor_cores", [1, 0])
def test_flash_decode_batch16_and_32k(cuda, oracle, name, tensor_cores):
    q, kc, vc, seq, slot, ref = _c3_case(oracle, name)
    B, Nq, D = q.shape
    cuda.set_tuning("flash_mma", tensor_cores)
    try:
        ws = cuda.flash_decode_workspace(B, Nq, D, kc.shape[2])
        out = cuda.flash_decode(q, kc, vc, dev(seq), dev(slot), workspace=ws).cpu().numpy()
    finally:
        cuda.set_tuning("flash_mma", FLASH_MMA_DEFAULT)
    err = rel_err(out, ref)
    assert err <= SPEC_TOL and err <= (5e-5 if tensor_cores else 1e-5)


@pytest.mark.parametrize("splits", [65, 100, 128])
def test_flash_decode_more_than_64_slices(cuda, oracle, splits):
    # calls of one or two rows may be cut into up to 128 slices per kv head (tensor-core kernel): the combining CTA then
    # holds four (max, sum) pairs per lane
    rng = np.random.default_rng(splits)
    B, Nq, Nkv, D, L = 2, 32, 8, 128, 9000
    q = rng.standard_normal((B, Nq, D)).astype(np.float32)
    kc = oracle.f32_to_bf16(rng.standard_normal((B, Nkv, L, D)).astype(np.float32))
    vc = oracle.f32_to_bf16(rng.standard_normal((B, Nkv, L, D)).astype(np.float32))
    seq = np.array([L, 8321], np.int32)
    slot = np.arange(B, dtype=np.int32)
    ref = oracle.attention(q, kc, vc, seq, slot)
    ws = cuda.flash_decode_workspace(B, Nq, D, L)
    cuda.set_tuning("flash_splits", splits)
    try:
        out = cuda.flash_decode(dev(q), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), dev(seq), dev(slot), workspace=ws).cpu().numpy()
    finally:
        cuda.set_tuning("flash_splits", 0)
    err = rel_err(out, ref)
    assert err <= SPEC_TOL and err <= 5e-5


def test_flash_decode_early_fetch_matches_conservative_path(cuda, oracle):
    # fresh_rows = F lets the kernel read cache rows below seq_len - F before the previous kernel has finished;
    # on a static cache both paths must give the same bits
    rng = np.random.default_rng(21)
    B, Nq, Nkv, D, Lmax = 3, 32, 8, 128, 2100
    kc = torch.randn((B, Nkv, Lmax, D), device="cuda").bfloat16()
    vc = torch.randn((B, Nkv, Lmax, D), device="cuda").bfloat16()
    q = dev(rng.standard_normal((B, Nq, D)).astype(np.float32))
    seq = dev(np.array([2084, 1, 700], np.int32))
    slot = dev(np.arange(B, dtype=np.int32))
    ws = cuda.flash_decode_workspace(B, Nq, D, Lmax)
    for mma in (0, 1):  # the SIMT kernel fetches ahead of the wait, the tensor-core kernel ignores the promise
        cuda.set_tuning("flash_mma", mma)
        try:
            ref = cuda.flash_decode(q, kc, vc, seq, slot, workspace=ws)
            for fresh in (0, 1, 3, 5000):
                got = cuda.flash_decode(q, kc, vc, seq, slot, workspace=ws, fresh_rows=fresh)
                torch.cuda.synchronize()
                assert torch.equal(got, ref), fresh
        finally:
            cuda.set_tuning("flash_mma", FLASH_MMA_DEFAULT)


@pytest.mark.parametrize("Nq,Nkv,lens,Lmax", [
    (32, 8, [2084, 1, 700], 2100), (16, 8, [65, 64], 2100), (8, 8, [130], 2100), (32, 8, [2084], 2100),
    (32, 8, [2048, 129], 2100), (64, 8, [1000], 2100),
    (32, 8, [4400], 4500),               # one sequence, eight-warp CTAs with two steps each
    (32, 8, [2305, 2304], 2400),         # two sequences, eight-warp CTAs, slices of uneven length
    (32, 8, [8200, 300, 5000], 9000),    # four-warp CTAs, many steps per slice (two register sets in flight)
    (32, 8, [20000], 20100)])            # one sequence past the eight-warp range: four-warp CTAs, one wave of slices
def test_rope_fused_into_flash_decode_is_bit_identical(cuda, oracle, Nq, Nkv, lens, Lmax):
    # decode batch: one row per slot, seq_len = pos + 1; the fused kernel must reproduce the two-kernel path bit for bit,
    # caches included, and may clear the raw projection rows and a side buffer
    rng = np.random.default_rng(31 + Nq)
    B, D = len(lens), 128
    kc = torch.randn((B, Nkv, Lmax, D), device="cuda").bfloat16()
    vc = torch.randn((B, Nkv, Lmax, D), device="cuda").bfloat16()
    kc2, vc2 = kc.clone(), vc.clone()
    qkv = dev(rng.standard_normal((B, (Nq + 2 * Nkv) * D)).astype(np.float32))
    qn = dev(oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32)))
    kn = dev(oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32)))
    cos_t, sin_t = (dev(t) for t in oracle.rope_tables(Lmax, D, 1e6))
    seq = dev(np.array(lens, np.int32))
    pos = dev(np.array(lens, np.int32) - 1)
    slot = dev(np.arange(B, dtype=np.int32))
    ws = cuda.flash_decode_workspace(B, Nq, D, Lmax)
    q = cuda.qknorm_rope_kvwrite(qkv.clone(), qn, kn, cos_t, sin_t, pos, slot, Nq, Nkv, D, 1e-6, kc, vc)
    cuda.set_tuning("flash_mma", 0)  # the fused kernel shares its arithmetic with the SIMT attention kernel
    try:
        ref = cuda.flash_decode(q, kc, vc, seq, slot, workspace=ws)
    finally:
        cuda.set_tuning("flash_mma", FLASH_MMA_DEFAULT)
    ref_mma = cuda.flash_decode(q, kc, vc, seq, slot, workspace=ws)
    assert rel_err(ref_mma.cpu().numpy(), ref.cpu().numpy()) <= 5e-5
    cuda.set_tuning("flash_mma_fused", 0)  # SIMT arithmetic in the fused kernel: bit-identical to the two SIMT kernels
    try:
        for fresh in (-1, 1):
            raw = qkv.clone()
            side = torch.ones((B, 512), device="cuda")
            k_f, v_f = kc2.clone(), vc2.clone()
            got = cuda.rope_flash_decode(raw, qn, kn, cos_t, sin_t, pos, seq, slot, Nq, Nkv, D, 1e-6, k_f, v_f, workspace=ws,
                                         fresh_rows=fresh, clear_input=True, clear_extra=side)
            torch.cuda.synchronize()
            assert torch.equal(got, ref), fresh
            assert torch.equal(k_f.view(torch.int16), kc.view(torch.int16)) and torch.equal(v_f.view(torch.int16), vc.view(torch.int16))
            assert float(raw.abs().max()) == 0.0 and float(side.abs().max()) == 0.0
    finally:
        cuda.set_tuning("flash_mma_fused", FLASH_MMA_FUSED_DEFAULT)
    # the same fused kernel with its contractions on the tensor cores: same caches and clearing, output to ~1e-5
    cuda.set_tuning("flash_mma_fused", 1)
    try:
        for fresh in (-1, 1):
            raw = qkv.clone()
            side = torch.ones((B, 512), device="cuda")
            k_f, v_f = kc2.clone(), vc2.clone()
            got = cuda.rope_flash_decode(raw, qn, kn, cos_t, sin_t, pos, seq, slot, Nq, Nkv, D, 1e-6, k_f, v_f, workspace=ws,
                                         fresh_rows=fresh, clear_input=True, clear_extra=side)
            torch.cuda.synchronize()
            assert rel_err(got.cpu().numpy(), ref.cpu().numpy()) <= 5e-5, fresh
            assert torch.equal(k_f.view(torch.int16), kc.view(torch.int16)) and torch.equal(v_f.view(torch.int16), vc.view(torch.int16))
            assert float(raw.abs().max()) == 0.0 and float(side.abs().max()) == 0.0
    finally:
        cuda.set_tuning("flash_mma_fused", FLASH_MMA_FUSED_DEFAULT)


def test_flash_decode_shared_cache_is_causal_prefill(cuda, oracle):
    # a prompt chunk: every row reads the same sequence, row i sees positions [0, i]
    rng = np.random.default_rng(9)
    M, Nq, Nkv, D, max_seq = 6, 16, 8, 128, 64
    q = rng.standard_normal((M, Nq, D)).astype(np.float32)
    kc = oracle.f32_to_bf16(rng.standard_normal((1, Nkv, max_seq, D)).astype(np.float32))
    vc = oracle.f32_to_bf16(rng.standard_normal((1, Nkv, max_seq, D)).astype(np.float32))
    seq = np.arange(10, 10 + M, dtype=np.int32)
    slot = np.zeros(M, np.int32)
    ref = oracle.attention(q, kc, vc, seq, slot)
    out = cuda.flash_decode(dev(q), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16), dev(seq), dev(slot)).cpu().numpy()
    assert rel_err(out, ref) <= 1e-5


# ----------------------------------------------------------------------------- tiled causal attention for prompt chunks
@pytest.mark.parametrize("M,pos0,Nq,Nkv", [(64, 0, 32, 8), (512, 0, 32, 8), (2048, 0, 32, 8), (100, 37, 16, 8), (70, 1000, 8, 8),
                                           (33, 5, 64, 8), (16, 0, 4, 2), (512, 1536, 32, 8)])
def test_flash_prefill_matches_oracle(cuda, oracle, M, pos0, Nq, Nkv):
    # a prompt chunk of M rows at positions pos0 .. pos0 + M - 1 of one sequence (slot 1 of 2): row m sees cache rows
    # [0, pos0 + m]; the oracle computes the same through its per-row attention
    rng = np.random.default_rng(M + pos0 + Nq)
    D = 128
    max_seq = pos0 + M + 3
    q = rng.standard_normal((M, Nq, D)).astype(np.float32)
    kc = oracle.f32_to_bf16(rng.standard_normal((2, Nkv, max_seq, D)).astype(np.float32))
    vc = oracle.f32_to_bf16(rng.standard_normal((2, Nkv, max_seq, D)).astype(np.float32))
    seq = (pos0 + 1 + np.arange(M)).astype(np.int32)
    slot = np.ones(M, np.int32)
    ref = oracle.attention(q, kc, vc, seq, slot)
    tq, tk, tv = dev(q), dev(kc, torch.bfloat16), dev(vc, torch.bfloat16)
    out = cuda.flash_prefill(tq, tk, tv, pos0, 1)
    again = cuda.flash_prefill(tq, tk, tv, pos0, 1)
    torch.cuda.synchronize()
    assert torch.equal(out, again)
    err = rel_err(out.cpu().numpy(), ref)
    assert err <= SPEC_TOL and err <= 5e-5   # 16 significant bits in q and in the probabilities
    # the per-row decode kernel on the same chunk: the two attention paths of the engine agree
    per_row = cuda.flash_decode(tq, tk, tv, dev(seq), dev(slot))
    torch.cuda.synchronize()
    assert rel_err(out.cpu().numpy(), per_row.cpu().numpy()) <= 1e-4


def test_flash_prefill_rejects_bad_arguments(cuda):
    from mykuiperllama_b200._lib import KuiperError
    q = torch.zeros((4, 8, 128), device="cuda")
    kc = torch.zeros((1, 2, 16, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(KuiperError) as e:
        cuda.flash_prefill(q, kc, kc, 14, 0)   # rows 14..17 exceed max_seq 16
    assert e.value.code == 7
    with pytest.raises(KuiperError) as e:
        cuda.flash_prefill(q, kc, kc, 0, 1)    # slot out of range
    assert e.value.code == 7


def test_rope_flash_decode_combine_wait_is_bounded(cuda, oracle):
    # eight-warp CTAs: the CTA of the last slice polls the other slices' words.  A slice that never sends (test hook) makes
    # the wait run out after the limit: the call returns, the status reports it once, and the next call is correct again
    from mykuiperllama_b200._lib import kernels
    lib = kernels()
    rng = np.random.default_rng(5)
    Nq, Nkv, D, Lmax, L = 32, 8, 128, 2100, 1500
    kc = torch.randn((1, Nkv, Lmax, D), device="cuda").bfloat16()
    vc = torch.randn((1, Nkv, Lmax, D), device="cuda").bfloat16()
    qkv = dev(rng.standard_normal((1, (Nq + 2 * Nkv) * D)).astype(np.float32))
    qn = dev(oracle.f32_to_bf16(np.ones(D, np.float32)))
    kn = dev(oracle.f32_to_bf16(np.ones(D, np.float32)))
    cos_t, sin_t = (dev(t) for t in oracle.rope_tables(Lmax, D, 1e6))
    seq, pos, slot = dev(np.array([L], np.int32)), dev(np.array([L - 1], np.int32)), dev(np.zeros(1, np.int32))
    ws = cuda.flash_decode_workspace(1, Nq, D, Lmax)

    def run():
        out = cuda.rope_flash_decode(qkv.clone(), qn, kn, cos_t, sin_t, pos, seq, slot, Nq, Nkv, D, 1e-6, kc.clone(), vc.clone(),
                                     workspace=ws, fresh_rows=1)
        torch.cuda.synchronize()
        return out

    assert lib.kuiper_flash_decode_status() == 0
    good = run()
    cuda.set_tuning("flash_timeout_ms", 50)
    cuda.set_tuning("flash_drop_slice", 3)
    try:
        run()
        assert lib.kuiper_flash_decode_status() == 5
        assert b"bounded wait" in lib.kuiper_last_error()
        assert lib.kuiper_flash_decode_status() == 0  # reported once
    finally:
        cuda.set_tuning("flash_drop_slice", -1)
        cuda.set_tuning("flash_timeout_ms", 1000)
    again = run()
    assert torch.equal(again, good)
    assert lib.kuiper_flash_decode_status() == 0


@pytest.mark.parametrize("lens,slots", [([2084], [2]), ([1500, 900], [1, 0]), ([2305, 64], [0, 2])])
def test_rope_flash_decode_with_rows_in_other_slots(cuda, oracle, lens, slots):
    # the eight-warp CTAs request their cache rows before slot[] has been read, guessing that row i sits in slot i; when
    # the guess is wrong they must fetch again - the result is that of the two-kernel path
    rng = np.random.default_rng(97 + len(lens))
    B, Nq, Nkv, D, Lmax, n_slots = len(lens), 32, 8, 128, 2400, 3
    kc = torch.randn((n_slots, Nkv, Lmax, D), device="cuda").bfloat16()
    vc = torch.randn((n_slots, Nkv, Lmax, D), device="cuda").bfloat16()
    qkv = dev(rng.standard_normal((B, (Nq + 2 * Nkv) * D)).astype(np.float32))
    qn = dev(oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32)))
    kn = dev(oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(D)).astype(np.float32)))
    cos_t, sin_t = (dev(t) for t in oracle.rope_tables(Lmax, D, 1e6))
    seq = dev(np.array(lens, np.int32))
    pos = dev(np.array(lens, np.int32) - 1)
    slot = dev(np.array(slots, np.int32))
    ws = cuda.flash_decode_workspace(B, Nq, D, Lmax)
    k_ref, v_ref = kc.clone(), vc.clone()
    q = cuda.qknorm_rope_kvwrite(qkv.clone(), qn, kn, cos_t, sin_t, pos, slot, Nq, Nkv, D, 1e-6, k_ref, v_ref)
    ref = cuda.flash_decode(q, k_ref, v_ref, seq, slot, workspace=ws)
    for fresh in (-1, 1):
        k_f, v_f = kc.clone(), vc.clone()
        got = cuda.rope_flash_decode(qkv.clone(), qn, kn, cos_t, sin_t, pos, seq, slot, Nq, Nkv, D, 1e-6, k_f, v_f, workspace=ws,
                                     fresh_rows=fresh)
        torch.cuda.synchronize()
        assert rel_err(got.cpu().numpy(), ref.cpu().numpy()) <= 5e-5, fresh
        assert torch.equal(k_f.view(torch.int16), k_ref.view(torch.int16)) and torch.equal(v_f.view(torch.int16), v_ref.view(torch.int16))


@pytest.mark.parametrize("M,K,N", [(16, 1024, 512), (48, 4096, 1024), (300, 2560, 4104)])
def test_fp16_activation_path_of_the_gemm(cuda, oracle, M, K, N):
    # the layer writes normalised / activated rows as fp16 straight into the GEMM's activation buffer: the results are
    # those of the fp32 kernels followed by the GEMM's own conversion pass, bit for bit (both round to nearest once)
    rng = np.random.default_rng(M + K)
    q, z, s = awq_random(rng, K, N)
    tqw, tqz, ts = dev(oracle.awq_pack(q)), dev(oracle.awq_pack(z)), dev(s.view(np.uint16), torch.float16)
    h = dev(rng.standard_normal((M, K)).astype(np.float32))
    nw = dev(oracle.f32_to_bf16((1 + 0.1 * rng.standard_normal(K)).astype(np.float32)))
    gu = dev(rng.standard_normal((M, 2 * K)).astype(np.float32))
    cuda.set_tuning("gemm_split_k", 0)  # fixed summation order, so that equality can be asserted
    try:
        x32 = cuda.rmsnorm(h, nw, 1e-6)
        x16 = cuda.rmsnorm_f16(h, nw, 1e-6)
        assert torch.equal(x16, x32.half())
        assert torch.equal(cuda.awq_gemm_f16in(x16, tqw, tqz, ts), cuda.awq_gemm(x32, tqw, tqz, ts))
        a32 = cuda.swiglu(gu.clone())
        a16 = cuda.swiglu_f16(gu.clone())
        assert torch.equal(a16, a32.half())
        res = dev(rng.standard_normal((M, N)).astype(np.float32))
        y1 = cuda.awq_gemm_f16in(a16, tqw, tqz, ts, y=res.clone(), accumulate=True)
        y2 = cuda.awq_gemm(a32, tqw, tqz, ts, y=res.clone(), accumulate=True)
        assert torch.equal(y1, y2)
    finally:
        cuda.set_tuning("gemm_split_k", 1)
    # with the K split the same call agrees to the summation order
    y3 = cuda.awq_gemm_f16in(x16, tqw, tqz, ts)
    torch.cuda.synchronize()
    assert rel_err(y3.cpu().numpy(), cuda.awq_gemm(x32, tqw, tqz, ts).cpu().numpy()) <= 2e-6
