"""Each CUDA kernel alone against a plain float32 torch restatement of the same operation
(``fake_ops.FakeOps`` on the CPU), at sizes other than the tiny engines': widths and vocabularies
that are no power of two, head sizes in steps of 16, odd head counts and page sizes.  Where random
data would hide a fault the inputs are constructed so that it shows (one far key that dominates,
the edge of a window, the last slot of a page)."""

from __future__ import annotations

import math

import pytest
import torch

import plain_qwen2 as plain
from fake_ops import FakeOps
from harness import assert_close
from mini_llm_runtime_b200 import ops
from mini_llm_runtime_b200.ops import cuda_ops
from mini_llm_runtime_b200.ops.cuda_ops import AttentionBatch, plan_attention

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
FAKE = FakeOps()


def cuda():
    return ops.current()


@pytest.fixture
def tcgen05_only():
    """Route few-row products to the tcgen05 kernel too (they default to the few-rows kernel)."""
    ops.current().use_skinny = False
    yield
    ops.current().use_skinny = True


def rnd(shape, dtype, seed, scale=1.0):
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=generator) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,width", [(1000, 100), (77, 896), (5, 3)])
def test_embedding(dtype, vocab, width):
    table = rnd((vocab, width), dtype, 1)
    ids = torch.randint(0, vocab, (37,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    got = cuda().embedding(ids.to(DEVICE), table.to(DEVICE))
    assert torch.equal(got.cpu(), FAKE.embedding(ids, table))
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32)
    assert torch.equal(cuda().gather_rows(got, rows.to(DEVICE)).cpu(), got.cpu()[rows.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,eps", [(100, 1e-6), (896, 1e-5), (5120, 1e-6), (7, 1e-3), (3584, 1e-6), (2056, 1e-5),
                                       (8192, 1e-6), (8200, 1e-6)])
def test_rms_norm_and_fused_add(dtype, width, eps):
    x = rnd((9, width), dtype, 3, 2.0)
    delta = rnd((9, width), dtype, 4, 0.5)
    weight = (1 + rnd((width,), torch.float32, 5, 0.1)).to(dtype)
    got = cuda().rms_norm(x.to(DEVICE), weight.to(DEVICE), eps)
    assert_close(got, plain.rms_norm(x, weight, eps), dtype, "rms_norm")
    residual = x.clone().to(DEVICE)
    got = cuda().add_rms_norm(residual, delta.to(DEVICE), weight.to(DEVICE), eps)
    summed = (x.float() + delta.float()).to(dtype)
    assert torch.equal(residual.cpu(), summed), "the residual must hold the once-rounded sum"
    assert_close(got, plain.rms_norm(summed, weight, eps), dtype, "add_rms_norm")


def test_rms_norm_keeps_a_float32_weight_with_bfloat16_rows():
    x = rnd((5, 200), torch.bfloat16, 6)
    weight = 1 + rnd((200,), torch.float32, 7, 0.1)
    got = cuda().rms_norm(x.to(DEVICE), weight.to(DEVICE), 1e-6)
    assert_close(got, plain.rms_norm(x, weight, 1e-6), torch.bfloat16, "rms_norm f32 weight")


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    gate_up = rnd((13, 2 * 203), dtype, 8, 3.0)
    got = cuda().swiglu(gate_up.to(DEVICE))
    assert_close(got, FAKE.swiglu(gate_up.float()), dtype, "swiglu")
    blocked = rnd((5, 2 * 192), dtype, 9, 3.0)
    got = cuda().swiglu(blocked.to(DEVICE), 64)
    assert_close(got, FAKE.swiglu(blocked.float(), 64), dtype, "swiglu, interleaved blocks")


def test_many_distinct_operands_never_share_a_tensor_map():
    """The tensor-core product looks its two tensor maps up in a host-side cache.  A model with more
    distinct matrices than the cache has entries (14B sizes: some four hundred) must still get the
    right map for each operand: with a cache that hands out pointers into its own table, the lookup
    of the second operand could overwrite the entry the first lookup had just returned."""
    generator = torch.Generator().manual_seed(77)
    weights = [(torch.randn(128 + 16 * (i % 5), 64 + 64 * (i % 3), generator=generator) * 0.2).to(torch.bfloat16).to(DEVICE)
               for i in range(700)]
    inputs = {k: (torch.randn(40, k, generator=generator)).to(torch.bfloat16).to(DEVICE) for k in (64, 128, 192)}
    for turn in range(2):                        # the second pass meets a full cache
        outputs = [cuda().linear(inputs[w.shape[1]], w) for w in weights]
        torch.cuda.synchronize()
        cuda().raise_if_device_error()
        for i in (0, 1, 255, 256, 257, 300, 511, 512, 699):
            want = inputs[weights[i].shape[1]].double() @ weights[i].double().T
            assert_close(outputs[i], want, torch.bfloat16, f"product {i}, pass {turn}")


@pytest.mark.parametrize("m", [1, 8, 20, 40, 100, 128, 200, 700])
@pytest.mark.parametrize("inner,k", [(4864, 896), (128, 64), (320, 200), (1216, 4864)])
def test_fused_linear_swiglu(m, inner, k, tcgen05_only):
    """The gate/up product with the activation in the tensor-core kernel's epilogue, in both
    orientations and with split-K, against the unfused float32 computation."""
    x = rnd((m, k), torch.bfloat16, 60 + m)
    gate = rnd((inner, k), torch.bfloat16, 61, 0.1)
    up = rnd((inner, k), torch.bfloat16, 62, 0.1)
    weight = torch.cat([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k)
    want = torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    got = cuda().linear_swiglu(x.to(DEVICE), weight.to(DEVICE), 64)
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    assert got.shape == (m, inner)
    assert_close(got, want, torch.bfloat16, f"fused linear+swiglu {m}x{inner}x{k}")
    cuda().use_fused_swiglu = False
    try:
        unfused = cuda().linear_swiglu(x.to(DEVICE), weight.to(DEVICE), 64)
    finally:
        cuda().use_fused_swiglu = True
    assert_close(unfused, want, torch.bfloat16, "unfused path on the interleaved layout")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 50, 17), (7, 130, 96), (33, 64, 300), (200, 203, 129), (16, 1, 1)])
def test_linear(dtype, m, n, k):
    x = rnd((m, k), dtype, 9)
    w = rnd((n, k), dtype, 10, 0.2)
    b = rnd((n,), dtype, 11)
    want = x.double() @ w.double().T + b.double()
    got = cuda().linear(x.to(DEVICE), w.to(DEVICE), b.to(DEVICE))
    assert_close(got, want, dtype, "linear+bias")
    got32 = cuda().linear(x.to(DEVICE), w.to(DEVICE), None, out_dtype=torch.float32)
    assert got32.dtype == torch.float32
    assert_close(got32, x.double() @ w.double().T, torch.float32 if dtype == torch.float32 else dtype, "linear f32 out")


@pytest.mark.parametrize("m,n,k", [(2048, 4864, 896), (1500, 2500, 200), (129, 151936 // 4, 72), (2048, 1216, 136),
                                   (3000, 1290, 4864)])
def test_many_row_products(m, n, k, tcgen05_only):
    """Prompt-sized products: more output tiles than SMs, tails in M, N and K, 128- and 256-wide
    tiles, with bias and with float32 output."""
    x = rnd((m, k), torch.bfloat16, 140 + m % 7)
    w = rnd((n, k), torch.bfloat16, 141, 0.1)
    b = rnd((n,), torch.bfloat16, 142)
    xd, wd, bd = x.to(DEVICE), w.to(DEVICE), b.to(DEVICE)
    want = x.double() @ w.double().T
    got = cuda().linear(xd, wd, bd)
    got32 = cuda().linear(xd, wd, None, out_dtype=torch.float32)
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    assert_close(got, want + b.double(), torch.bfloat16, f"many rows {m}x{n}x{k}")
    assert float((got32.double().cpu() - want).abs().max()) <= 1e-4 * float(want.abs().max()) + 1e-5


@pytest.mark.parametrize("m,n,k", [(600, 300, 72), (1000, 1290, 3584), (512, 256, 64), (2049, 896, 200)])
def test_two_accumulators_per_cta(m, n, k, tcgen05_only):
    """The 256 x 256 tile plan (two 128-row accumulators side by side in tensor memory from one load
    of the weight tile), forced through the kernel's debug entry: tails in M (the second accumulator
    partly or wholly empty), N and K; plain, float32 and SwiGLU epilogues."""
    from mini_llm_runtime_b200.ops import build

    lib = build.load_library("gemm_tcgen05")
    x = rnd((m, k), torch.bfloat16, 170 + m % 5)
    w = rnd((n, k), torch.bfloat16, 171, 0.1)
    b = rnd((n,), torch.bfloat16, 172)
    inner = (n // 128) * 64
    xd, wd, bd = x.to(DEVICE), w.to(DEVICE), b.to(DEVICE)
    lib.mlr_gemm_tcgen05_debug(256, 0, 1, 256)
    try:
        got = cuda().linear(xd, wd, bd)
        got32 = cuda().linear(xd, wd, None, out_dtype=torch.float32)
        if inner >= 128:
            gate = rnd((inner, k), torch.bfloat16, 173, 0.1)
            up = rnd((inner, k), torch.bfloat16, 174, 0.1)
            stacked = torch.cat([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k)
            act = cuda().linear_swiglu(xd, stacked.to(DEVICE), 64)
        torch.cuda.synchronize()
        cuda().raise_if_device_error()
    finally:
        lib.mlr_gemm_tcgen05_debug(0, 0, 0, 0)
    want = x.double() @ w.double().T
    assert_close(got, want + b.double(), torch.bfloat16, f"256 x 256 tiles {m}x{n}x{k}")
    assert float((got32.double().cpu() - want).abs().max()) <= 1e-4 * float(want.abs().max()) + 1e-5
    if inner >= 128:
        assert_close(act, torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T),
                     torch.bfloat16, "256 x 256 tiles with SwiGLU")


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("m,n,k", [(600, 300, 72), (1000, 1290, 3584), (257, 256, 64), (2049, 896, 200)])
def test_tile_over_an_sm_pair(m, n, k, mode, tcgen05_only):
    """The 256 x 256 tile over a cluster of two CTAs (each loads its 128 rows and half of the weight
    rows; one thread of the even CTA issues MMAs for both; commits arrive in both), forced through
    the debug entry with long rings (one CTA per SM) and short ones (two): tails in M (the odd CTA
    partly or wholly empty), N (the odd CTA's weight half partly or wholly outside) and K; plain,
    float32 and SwiGLU epilogues; and the same bits as the tile computed by one CTA."""
    from mini_llm_runtime_b200.ops import build

    lib = build.load_library("gemm_tcgen05")
    x = rnd((m, k), torch.bfloat16, 180 + m % 5)
    w = rnd((n, k), torch.bfloat16, 181, 0.1)
    b = rnd((n,), torch.bfloat16, 182)
    inner = (n // 128) * 64
    xd, wd, bd = x.to(DEVICE), w.to(DEVICE), b.to(DEVICE)
    lib.mlr_gemm_tcgen05_debug_pair(-1)
    lib.mlr_gemm_tcgen05_debug(256, 0, 1, 128)
    try:
        alone = cuda().linear(xd, wd, bd)
        lib.mlr_gemm_tcgen05_debug(0, 0, 0, 0)
        lib.mlr_gemm_tcgen05_debug_pair(mode)
        got = cuda().linear(xd, wd, bd)
        got32 = cuda().linear(xd, wd, None, out_dtype=torch.float32)
        if inner >= 128:
            gate = rnd((inner, k), torch.bfloat16, 183, 0.1)
            up = rnd((inner, k), torch.bfloat16, 184, 0.1)
            stacked = torch.cat([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k)
            act = cuda().linear_swiglu(xd, stacked.to(DEVICE), 64)
        torch.cuda.synchronize()
        cuda().raise_if_device_error()
    finally:
        lib.mlr_gemm_tcgen05_debug(0, 0, 0, 0)
        lib.mlr_gemm_tcgen05_debug_pair(0)
    want = x.double() @ w.double().T
    assert torch.equal(got, alone), "an SM pair and one CTA differ"
    assert_close(got, want + b.double(), torch.bfloat16, f"SM pair {m}x{n}x{k}")
    assert float((got32.double().cpu() - want).abs().max()) <= 1e-4 * float(want.abs().max()) + 1e-5
    if inner >= 128:
        assert_close(act, torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T),
                     torch.bfloat16, "SM pair with SwiGLU")


@pytest.mark.parametrize("m,inner,k", [(2048, 4864, 896), (777, 1216, 200), (1300, 2560, 4864)])
def test_many_row_swiglu(m, inner, k, tcgen05_only):
    x = rnd((m, k), torch.bfloat16, 150)
    gate = rnd((inner, k), torch.bfloat16, 151, 0.1)
    up = rnd((inner, k), torch.bfloat16, 152, 0.1)
    weight = torch.cat([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k)
    want = torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    got = cuda().linear_swiglu(x.to(DEVICE), weight.to(DEVICE), 64)
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    assert_close(got, want, torch.bfloat16, f"many-row fused linear+swiglu {m}x{inner}x{k}")


@pytest.mark.parametrize("m", [1, 8, 16, 17, 33, 64, 100, 128, 129, 300])
@pytest.mark.parametrize("n,k", [(896, 896), (1152, 896), (200, 72), (896, 4864), (130, 64), (4000, 136)])
def test_tensor_core_linear(m, n, k, tcgen05_only):
    """The tcgen05 product in both orientations, with and without split-K, K tails and N tails."""
    x = rnd((m, k), torch.bfloat16, 40 + m)
    w = rnd((n, k), torch.bfloat16, 41, 0.1)
    b = rnd((n,), torch.bfloat16, 42)
    want = x.double() @ w.double().T + b.double()
    got = cuda().linear(x.to(DEVICE), w.to(DEVICE), b.to(DEVICE))
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    assert_close(got, want, torch.bfloat16, f"tcgen05 linear {m}x{n}x{k}")
    # float32 output keeps the accumulator's precision: far tighter than bfloat16 rounding
    got32 = cuda().linear(x.to(DEVICE), w.to(DEVICE), None, out_dtype=torch.float32)
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    want32 = x.double() @ w.double().T
    assert float((got32.double().cpu() - want32).abs().max()) <= 1e-4 * float(want32.abs().max()) + 1e-5
    # and it is the same bits when called again (split-K partials are added in a fixed order)
    assert torch.equal(got32, cuda().linear(x.to(DEVICE), w.to(DEVICE), None, out_dtype=torch.float32))


@pytest.mark.parametrize("m,n,k", [(2048, 4864, 896), (1000, 896, 4864), (2048, 1152, 896), (517, 5000, 264)])
def test_tensor_core_linear_many_rows(m, n, k):
    """Prefill-sized products: 128x128 and 128x256 tiles, ragged edges in every dimension."""
    x = rnd((m, k), torch.bfloat16, 70)
    w = rnd((n, k), torch.bfloat16, 71, 0.05)
    b = rnd((n,), torch.bfloat16, 72)
    got = cuda().linear(x.to(DEVICE), w.to(DEVICE), b.to(DEVICE))
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    want = (x.to(DEVICE).double() @ w.to(DEVICE).double().T + b.to(DEVICE).double()).cpu()
    assert_close(got, want, torch.bfloat16, f"tcgen05 linear {m}x{n}x{k}")


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(896, 896), (1152, 896), (896, 4864), (200, 72), (130, 64), (4000, 136), (5120, 5120),
                                 (520, 3584), (72, 2056), (99, 4360)])
def test_few_rows_linear(m, n, k):
    """The few-rows kernel (mma.sync on 16-row weight groups, K shared by the CTA's warps) against
    float64, and against the tcgen05 kernel on the same inputs."""
    x = rnd((m, k), torch.bfloat16, 90 + m)
    w = rnd((n, k), torch.bfloat16, 91, 0.1)
    b = rnd((n,), torch.bfloat16, 92)
    want = x.double() @ w.double().T + b.double()
    cuda().SKINNY_ROWS = 64          # the kernel takes up to 64 rows; the dispatcher stops at 16
    cuda().skinny_one_round = False  # and leaves grids of more than one round to the tcgen05 kernel
    try:
        _check_few_rows(m, n, k, x, w, b, want)
    finally:
        del cuda().SKINNY_ROWS
        del cuda().skinny_one_round


def test_few_rows_kernel_is_left_when_its_grid_takes_more_than_one_round():
    """The dispatcher asks the few-rows kernel in how many rounds its CTAs would run (the device's own
    occupancy figure) and, with more than one token row and a matrix of megabytes, gives a grid of
    more than one round to the tcgen05 kernel; the answer does not change the result."""
    ops_ = cuda()
    assert ops_._skinny_rounds(8, 1152, 896, False) == 1            # 72 CTAs
    assert ops_._skinny_rounds(8, 9728, 896, True) == 1             # 304 CTAs, three per SM
    wide = 16 * (2 * ops_.sm_count(torch.device(DEVICE)) + 8)       # 8 warps per CTA, two CTAs per SM: 8 CTAs too many
    assert ops_._skinny_rounds(8, wide, 5120, False) >= 2
    x = rnd((8, 5120), torch.bfloat16, 410)
    w = rnd((wide, 5120), torch.bfloat16, 411, 0.1)
    xd, wd = x.to(DEVICE), w.to(DEVICE)
    assert not ops_._skinny_fits(xd, wd) and ops_._skinny_fits(xd[:1], wd)
    by_rule = ops_.linear(xd, wd)
    ops_.skinny_one_round = False
    try:
        assert ops_._skinny_fits(xd, wd)
        few_rows = ops_.linear(xd, wd)
    finally:
        del ops_.skinny_one_round
    want = x.double() @ w.double().T
    assert_close(by_rule, want, torch.bfloat16, "the tcgen05 kernel by the one-round rule")
    assert_close(few_rows, want, torch.bfloat16, "the few-rows kernel in rounds")


def _check_few_rows(m, n, k, x, w, b, want):
    assert cuda()._skinny_fits(x, w)
    got = cuda().linear(x.to(DEVICE), w.to(DEVICE), b.to(DEVICE))
    assert_close(got, want, torch.bfloat16, f"few-rows linear {m}x{n}x{k}")
    got32 = cuda().linear(x.to(DEVICE), w.to(DEVICE), None, out_dtype=torch.float32)
    want32 = x.double() @ w.double().T
    assert float((got32.double().cpu() - want32).abs().max()) <= 1e-4 * float(want32.abs().max()) + 1e-5
    assert torch.equal(got32, cuda().linear(x.to(DEVICE), w.to(DEVICE), None, out_dtype=torch.float32))
    cuda().use_skinny = False
    try:
        other = cuda().linear(x.to(DEVICE), w.to(DEVICE), b.to(DEVICE))
    finally:
        cuda().use_skinny = True
    assert_close(got, other, torch.bfloat16, "few-rows kernel against the tcgen05 kernel")


@pytest.mark.parametrize("m", [1, 7, 16, 30, 64])
@pytest.mark.parametrize("n,k,eps", [(896, 4864, 1e-6), (1152, 896, 1e-5), (100, 72, 1e-3), (24, 4104, 1e-6), (40, 3584, 1e-6), (99, 4360, 1e-6)])
def test_few_rows_linear_with_norm_and_residual(m, n, k, eps):
    """The row scale of an RMS norm taken inside the product, and the result added into a residual
    in place; alone and together, against the same operations done separately in float64.  The
    same calls through the many-rows kernels (norm kernel, product, add kernel) must agree."""
    x = rnd((m, k), torch.bfloat16, 300 + m, 3.0)
    x[m // 2] *= 40.0                               # rows of very different size: each needs its own scale
    w = rnd((n, k), torch.bfloat16, 301, 0.1)
    b = rnd((n,), torch.bfloat16, 302)
    base = rnd((m, n), torch.bfloat16, 303, 2.0)
    xd = x.double()
    normed = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + eps)
    cuda().SKINNY_ROWS = 64
    cuda().skinny_one_round = False
    try:
        assert cuda()._skinny_fits(x.to(DEVICE), w.to(DEVICE)) and cuda().fuses_norm(m)
        for skinny in (True, False):
            cuda().use_skinny = skinny
            got = cuda().linear(x.to(DEVICE), w.to(DEVICE), b.to(DEVICE), rms_eps=eps)
            assert_close(got, normed @ w.double().T + b.double(), torch.bfloat16, f"norm inside the product, few-rows={skinny}")
            stream = base.clone().to(DEVICE)
            got = cuda().linear(x.to(DEVICE), w.to(DEVICE), None, residual=stream)
            assert got.data_ptr() == stream.data_ptr()
            assert_close(got, base.double() + xd @ w.double().T, torch.bfloat16, f"residual add, few-rows={skinny}")
            stream = base.clone().to(DEVICE)
            cuda().linear(x.to(DEVICE), w.to(DEVICE), b.to(DEVICE), rms_eps=eps, residual=stream)
            assert_close(stream, base.double() + normed @ w.double().T + b.double(), torch.bfloat16,
                         f"norm and residual, few-rows={skinny}")
    finally:
        cuda().use_skinny = True
        del cuda().SKINNY_ROWS
        del cuda().skinny_one_round


@pytest.mark.parametrize("m", [2, 16, 40])
def test_few_rows_linear_swiglu_with_norm(m):
    inner, k, eps = 320, 200, 1e-6
    x = rnd((m, k), torch.bfloat16, 310 + m, 5.0)
    gate = rnd((inner, k), torch.bfloat16, 311, 0.1)
    up = rnd((inner, k), torch.bfloat16, 312, 0.1)
    weight = torch.cat([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k)
    xd = x.double()
    normed = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + eps)
    want = torch.nn.functional.silu(normed @ gate.double().T) * (normed @ up.double().T)
    cuda().SKINNY_ROWS = 64
    try:
        for skinny in (True, False):
            cuda().use_skinny = skinny
            got = cuda().linear_swiglu(x.to(DEVICE), weight.to(DEVICE), 64, rms_eps=eps)
            assert_close(got, want, torch.bfloat16, f"norm inside the fused gate/up product, few-rows={skinny}")
    finally:
        cuda().use_skinny = True
        del cuda().SKINNY_ROWS


@pytest.mark.parametrize("dtype", DTYPES)
def test_weightless_norm_and_add_inplace(dtype):
    x = rnd((9, 200), dtype, 320, 2.0)
    delta = rnd((9, 200), dtype, 321)
    got = cuda().rms_norm(x.to(DEVICE), None, 1e-5)
    assert_close(got, plain.rms_norm(x, torch.ones(200), 1e-5), dtype, "norm without a weight")
    target = x.clone().to(DEVICE)
    assert cuda().add_inplace(target, delta.to(DEVICE)).data_ptr() == target.data_ptr()
    assert torch.equal(target.cpu(), (x.float() + delta.float()).to(dtype))
    target = x.clone().to(DEVICE)
    got = cuda().add_rms_norm(target, delta.to(DEVICE), None, 1e-5)
    assert_close(got, plain.rms_norm((x.float() + delta.float()).to(dtype), torch.ones(200), 1e-5), dtype, "add + weightless norm")


@pytest.mark.parametrize("m", [1, 8, 13, 30, 64])
@pytest.mark.parametrize("inner,k", [(4864, 896), (128, 64), (320, 200)])
def test_few_rows_linear_swiglu(m, inner, k):
    x = rnd((m, k), torch.bfloat16, 95 + m)
    gate = rnd((inner, k), torch.bfloat16, 96, 0.1)
    up = rnd((inner, k), torch.bfloat16, 97, 0.1)
    weight = torch.cat([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inner, k)
    want = torch.nn.functional.silu(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    cuda().SKINNY_ROWS = 64
    try:
        assert cuda()._skinny_fits(x, weight, swiglu=True)
        got = cuda().linear_swiglu(x.to(DEVICE), weight.to(DEVICE), 64)
    finally:
        del cuda().SKINNY_ROWS
    assert got.shape == (m, inner)
    assert_close(got, want, torch.bfloat16, f"few-rows fused gate/up {m}x{inner}x{k}")


def test_tensor_core_linear_large_vocabulary():
    x = rnd((8, 896), torch.bfloat16, 50)
    w = rnd((151936, 896), torch.bfloat16, 51, 0.02)
    got = cuda().linear(x.to(DEVICE), w.to(DEVICE), None, out_dtype=torch.float32)
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    want = x.double() @ w.double().T
    assert float((got.double().cpu() - want).abs().max()) <= 1e-4 * float(want.abs().max()) + 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_rows_do_not_depend_on_the_batch(dtype):
    x = rnd((70, 152), dtype, 12).to(DEVICE)
    w = rnd((90, 152), dtype, 13, 0.2).to(DEVICE)
    whole = cuda().linear(x, w)
    for start, stop in [(0, 1), (5, 22), (69, 70), (16, 70)]:
        assert torch.equal(cuda().linear(x[start:stop].contiguous(), w), whole[start:stop])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(5, 1, 16, 4), (6, 3, 48, 16), (4, 4, 128, 8), (2, 1, 256, 3)])
def test_rope_and_cache_write(dtype, heads, kv_heads, head_dim, page):
    tokens, pages = 11, 9
    theta = 1000000.0
    qkv = rnd((tokens, (heads + 2 * kv_heads) * head_dim), dtype, 14)
    positions = torch.tensor([0, 1, 2, 3, 500, 4095, 7, 31999, 8, 9, 10], dtype=torch.int32)
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    # last slot of a page, first slot of a page, one padding row (-1), scattered pages
    slots = torch.tensor([page - 1, page, -1, 5 * page + 1, 0, 8 * page + page - 1, 2 * page, 3 * page + 1,
                          4 * page, 6 * page, 7 * page], dtype=torch.int64)
    k_ref = torch.full((pages, kv_heads, page, head_dim), 7.0).to(dtype)
    v_ref = torch.full((pages, kv_heads, page, head_dim), -7.0).to(dtype)
    k_dev, v_dev = k_ref.clone().to(DEVICE), v_ref.clone().to(DEVICE)
    q_ref = FAKE.rope_kv_write(qkv.float(), positions, inv_freq, slots, k_ref, v_ref, heads, kv_heads, head_dim)
    q_dev = cuda().rope_kv_write(qkv.to(DEVICE), positions.to(DEVICE), inv_freq.to(DEVICE), slots.to(DEVICE),
                                 k_dev, v_dev, heads, kv_heads, head_dim)
    assert_close(q_dev, q_ref, dtype, "rotated q")
    assert_close(k_dev.reshape(pages, -1), k_ref.reshape(pages, -1), dtype, "k pages (untouched slots included)")
    assert torch.equal(v_dev.cpu(), v_ref), "v is copied unrotated and bit-exact"
    # write_kv=False leaves the pages alone
    k_before = k_dev.clone()
    cuda().rope_kv_write(qkv.to(DEVICE), positions.to(DEVICE), inv_freq.to(DEVICE), slots.to(DEVICE),
                         k_dev, v_dev, heads, kv_heads, head_dim, write_kv=False)
    assert torch.equal(k_dev, k_before)


def make_attention_case(dtype, heads, kv_heads, head_dim, page, segments, seed, pages_total=None):
    """segments: list of (pos0, q_len).  Pages are handed out in a scrambled order; every slot
    that no request owns is poisoned with NaN so that a stray read shows."""
    generator = torch.Generator().manual_seed(seed)
    need = [-(-(pos0 + q_len) // page) for pos0, q_len in segments]
    pages_total = pages_total or sum(need) + 3
    order = torch.randperm(pages_total, generator=generator).tolist()
    width = max(need)
    table = torch.full((len(segments), width), -1, dtype=torch.int32)
    k_pool = torch.full((pages_total, kv_heads, page, head_dim), float("nan"))
    v_pool = torch.full((pages_total, kv_heads, page, head_dim), float("nan"))
    cursor = 0
    for s, (pos0, q_len) in enumerate(segments):
        for logical in range(need[s]):
            table[s, logical] = order[cursor]
            cursor += 1
        for t in range(pos0 + q_len):
            pg, off = table[s, t // page], t % page
            k_pool[pg, :, off] = torch.randn(kv_heads, head_dim, generator=generator)
            v_pool[pg, :, off] = torch.randn(kv_heads, head_dim, generator=generator)
    rows = sum(q for _, q in segments)
    q = torch.randn(rows, heads * head_dim, generator=generator)
    q_start, row = [], 0
    for _, q_len in segments:
        q_start.append(row)
        row += q_len
    lengths = [q_len for _, q_len in segments]
    starts = [pos0 for pos0, _ in segments]
    arrays, counts = plan_attention(lengths, starts)

    def ints(values, device):
        return torch.tensor(values, dtype=torch.int32, device=device)

    def batch(device):
        return AttentionBatch(
            seg_q_start=ints(q_start, device), seg_q_len=ints(lengths, device), seg_pos0=ints(starts, device),
            seg_slot=ints(list(range(len(segments))), device), block_table=table.to(device),
            num_segments=len(segments), max_q_len=max(lengths), max_kv_len=max(p + q for p, q in segments),
            plan={name: torch.from_numpy(array).to(device) for name, array in arrays.items()}, counts=counts)

    return q.to(dtype), k_pool.to(dtype), v_pool.to(dtype), batch, table


def run_attention_both(dtype, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window):
    scale = head_dim ** -0.5
    want = FAKE.paged_attention(q.float(), k_pool.float(), v_pool.float(), batch("cpu"), heads, kv_heads,
                                head_dim, scale, window)
    got = cuda().paged_attention(q.to(DEVICE), k_pool.to(DEVICE), v_pool.to(DEVICE), batch(DEVICE), heads,
                                 kv_heads, head_dim, scale, window)
    return got, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [
    (14, 2, 64, 16), (3, 1, 32, 8), (6, 3, 48, 16), (8, 8, 128, 16), (2, 1, 256, 3), (5, 5, 16, 4), (4, 2, 80, 32)])
def test_attention_ragged_batch(dtype, heads, kv_heads, head_dim, page):
    # a whole prompt, a portion in the middle of a request, two single decoded tokens, a 2-token portion
    segments = [(0, 37), (50, 19), (130, 1), (0, 1), (63, 2)]
    q, k_pool, v_pool, batch, _ = make_attention_case(dtype, heads, kv_heads, head_dim, page, segments, 21)
    got, want = run_attention_both(dtype, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
    assert_close(got, want, dtype, "attention")


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(14, 2, 64, 16), (3, 1, 128, 8), (8, 8, 64, 16), (8, 1, 128, 32), (5, 1, 64, 3),
                                                          (4, 2, 64, 64), (7, 1, 128, 128), (2, 2, 64, 256), (6, 2, 64, 4)])
@pytest.mark.parametrize("chunk", [None, 128, 512])
def test_decode_attention_split_kv(heads, kv_heads, head_dim, page, chunk):
    """Single-row segments go through the split-KV kernel: contexts around the warp (32), CTA (128)
    and chunk boundaries, beside a prompt portion that takes the other kernel."""
    contexts = [0, 1, 30, 31, 32, 33, 126, 127, 128, 129, 255, 256, 511, 512, 513, 700, 1500]
    segments = [(c, 1) for c in contexts[:9]] + [(40, 21)] + [(c, 1) for c in contexts[9:]]
    q, k_pool, v_pool, batch, _ = make_attention_case(torch.bfloat16, heads, kv_heads, head_dim, page, segments, 25)
    cuda().decode_chunk = chunk
    try:
        for window in (None, 100):
            got, want = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
            assert_close(got, want, torch.bfloat16, f"decode attention chunk={chunk} window={window}")
            again, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
            assert torch.equal(got, again), "chunks are merged in a fixed order: same bits every time"
            # pages of 8 keys or more (a power of two) go to the kernel that loads by bulk tensor copies
            cuda().use_tma_attention = False
            try:
                other, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
            finally:
                cuda().use_tma_attention = True
            assert_close(got, other, torch.bfloat16, "bulk-copy kernel against the cp.async kernel")
    finally:
        cuda().decode_chunk = None
    cuda().use_decode_kernel = False
    cuda().use_mma_attention = False
    try:
        generic, want = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
        cuda().use_decode_kernel = True
        simt, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
    finally:
        cuda().use_decode_kernel = True
        cuda().use_mma_attention = True
    assert_close(generic, want, torch.bfloat16, "generic kernel")
    assert_close(simt, want, torch.bfloat16, "split-KV kernel on the CUDA cores")
    both, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
    assert_close(both, generic, torch.bfloat16, "tensor-core kernels against the generic kernel")


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(14, 2, 64, 16), (28, 4, 128, 16), (5, 1, 128, 64)])
def test_decode_attention_merges_through_clusters_of_every_size(heads, kv_heads, head_dim, page):
    """Contexts of up to 4,096 keys for few requests: the chunks of a (request, kv head) form a
    thread-block cluster of 2 to 16 CTAs (by the number of pairs and the longest context) that merges through shared
    memory.  Short contexts in the same launch leave most of their cluster's CTAs without keys;
    one far key is made dominant so that a chunk merged with the wrong weight shows.  Against the
    plain stand-in and against the merge through scratch memory."""
    contexts_by_rows = {4: [4095, 100, 2600, 257], 9: [4000, 3, 255, 256, 1023, 3071, 2048, 64, 700],
                        5: [1000, 3, 700, 256, 999], 6: [2047, 80, 1025, 512, 1900, 71],     # clusters of 6 and of 8
                        20: [4095] + [137 * i % 3900 + 1 for i in range(19)],
                        28: [4095] + [211 * i % 4000 + 1 for i in range(27)]}
    for rows, contexts in contexts_by_rows.items():
        if rows * kv_heads > cuda().clusters_together(3):     # more pairs than even clusters of 3 run together
            continue
        segments = [(c, 1) for c in contexts]
        q, k_pool, v_pool, batch, table = make_attention_case(torch.bfloat16, heads, kv_heads, head_dim, page, segments, 70 + rows)
        direction = q[0, :head_dim].float()                      # request 0, head 0: key 70 dominates
        pg, off = table[0, 70 // page], 70 % page
        k_pool[pg, 0, off] = (direction * (40.0 / direction.norm() ** 2 * math.sqrt(head_dim))).to(torch.bfloat16)
        v_pool[pg, 0, off] = torch.full((head_dim,), 100.0).to(torch.bfloat16)
        got, want = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
        torch.cuda.synchronize()
        cuda().raise_if_device_error()
        assert_close(got, want, torch.bfloat16, f"decode attention, {rows} rows, cluster merge")
        assert float(got[0, :head_dim].float().mean()) > 90.0, "the dominant far key was lost"
        again, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
        assert torch.equal(got, again), "chunks are merged in chunk order: same bits every time"
        cuda().use_cluster_merge = False
        try:
            other, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
        finally:
            cuda().use_cluster_merge = True
        assert_close(got, other, torch.bfloat16, "cluster merge against the merge through scratch memory")


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(14, 2, 64, 16), (3, 1, 128, 8), (8, 8, 64, 64), (8, 2, 128, 32), (5, 1, 64, 256)])
@pytest.mark.parametrize("write_kv", [True, False])
def test_decode_attention_with_fused_position_encoding(heads, kv_heads, head_dim, page, write_kv):
    """A step of decoded tokens only: rotation of q and k, the cache write and attention in one
    kernel, against the two kernels it replaces.  Rotated values are rounded the same way in both,
    so outputs and pages must agree to the bit.  Contexts sit on tile, page and chunk edges."""
    contexts = [0, 1, 31, 32, 63, 64, 65, 127, 255, 256, 511, 512, 513, 700, 1500, 2047]
    segments = [(c, 1) for c in contexts]
    q, k_pool, v_pool, batch, table = make_attention_case(torch.bfloat16, heads, kv_heads, head_dim, page, segments, 31)
    k_pool, v_pool = torch.nan_to_num(k_pool, nan=3.0), torch.nan_to_num(v_pool, nan=-3.0)   # pages are compared whole
    qkv = rnd((len(contexts), (heads + 2 * kv_heads) * head_dim), torch.bfloat16, 32)
    positions = torch.tensor(contexts, dtype=torch.int32)
    slots = torch.tensor([int(table[s, c // page]) * page + c % page for s, c in enumerate(contexts)], dtype=torch.int64)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    results = {}
    for fused in (False, True, "32-key tiles"):
        if fused == "32-key tiles" and head_dim != 64:
            continue
        k_dev, v_dev = k_pool.clone().to(DEVICE), v_pool.clone().to(DEVICE)
        cuda().use_fused_rope = bool(fused)
        cuda().decode_stages = 12 if fused == "32-key tiles" else None      # 32-key tiles, two in flight per warp
        try:
            for window in (None, 100):
                before = cuda_ops.launches
                out = cuda().rope_paged_attention(qkv.to(DEVICE), positions.to(DEVICE), inv_freq.to(DEVICE),
                                                  slots.to(DEVICE), k_dev, v_dev, batch(DEVICE), heads, kv_heads,
                                                  head_dim, head_dim ** -0.5, window, write_kv)
                assert cuda_ops.launches - before == (1 if fused else 2)
                results[fused, window] = out
        finally:
            cuda().use_fused_rope = True
            cuda().decode_stages = None
        results[fused, "k"], results[fused, "v"] = k_dev, v_dev
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    for key in (None, 100, "k", "v"):
        assert torch.equal(results[True, key], results[False, key]), f"fused and separate kernels differ in {key}"
    if head_dim == 64:
        for key in ("k", "v"):
            assert torch.equal(results["32-key tiles", key], results[False, key]), "pages written with 32-key tiles differ"
        for key in (None, 100):
            assert_close(results["32-key tiles", key], results[True, key], torch.bfloat16, "32-key tiles against 64-key tiles")
    if not write_kv:
        assert torch.equal(results[True, "k"].cpu(), k_pool) and torch.equal(results[True, "v"].cpu(), v_pool)
    # and against the plain stand-in, which rotates and attends in float32
    k_ref, v_ref = k_pool.clone().float(), v_pool.clone().float()
    want = FAKE.rope_paged_attention(qkv.float(), positions, inv_freq, slots, k_ref, v_ref, batch("cpu"), heads, kv_heads,
                                     head_dim, head_dim ** -0.5, None, write_kv)
    assert_close(results[True, None], want, torch.bfloat16, "fused position encoding and attention")


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(14, 2, 64, 16), (4, 1, 128, 8), (6, 6, 64, 32), (16, 1, 128, 16),
                                                          (2, 1, 64, 64), (3, 3, 128, 128), (4, 2, 64, 4)])
@pytest.mark.parametrize("window", [None, 70])
def test_prefill_attention_tensor_cores(heads, kv_heads, head_dim, page, window):
    """Prompt portions through the tensor-core kernel: a whole prompt longer than several tiles,
    portions that start in the middle of a request (at and off tile and page edges), very short
    portions, beside decoded tokens."""
    segments = [(0, 300), (64, 64), (100, 130), (63, 2), (500, 1), (0, 1), (127, 65), (5, 3)]
    q, k_pool, v_pool, batch, _ = make_attention_case(torch.bfloat16, heads, kv_heads, head_dim, page, segments, 26)
    got, want = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
    assert_close(got, want, torch.bfloat16, f"prefill attention window={window}")
    again, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
    assert torch.equal(got, again), "tiles drawn from the queue in any order give the same bits"
    # tiles loaded by cp.async and one CTA per tile (the compiler contracts the unmasked softmax of
    # interior tiles differently, so the two agree to rounding, not to the bit)
    cuda().use_tma_attention = cuda().use_tcgen05_attention = False
    try:
        other, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
    finally:
        cuda().use_tma_attention = cuda().use_tcgen05_attention = True
    assert_close(got, other, torch.bfloat16, "default prefill kernel against the cp.async prefill kernel")
    # pages of 8 keys or more took the tcgen05 kernel above (S = Q K^T and P V in tensor memory, one
    # thread per query row); the mma.sync kernel with bulk-copy loaders must agree with it
    cuda().use_tcgen05_attention = False
    try:
        third, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
        torch.cuda.synchronize()
        cuda().raise_if_device_error()
    finally:
        cuda().use_tcgen05_attention = True
    assert_close(third, want, torch.bfloat16, f"mma.sync prefill attention window={window}")
    assert_close(third, got, torch.bfloat16, "mma.sync prefill kernel against the default kernel")


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("rises", [(5.0, 12.0, 14.0, 30.0, 33.0), (40.0, 41.0, 3.0, 2.0, 1.0), (4.0, 4.5, 5.0, 5.5, 6.0)])
def test_prefill_attention_rising_maxima(head_dim, rises):
    """The tcgen05 kernel keeps the output rows in tensor memory relative to a base exponent that
    follows the running max only in steps of more than 2^8.  Keys in five different key tiles are
    given scores that rise by small and by large amounts for the last row of the prompt, so that
    some tiles move the base (the rows are rescaled in tensor memory) and others run ahead of it."""
    heads, kv_heads, page = 3, 1, 16
    segments = [(0, 700), (300, 140)]
    q, k_pool, v_pool, batch, table = make_attention_case(torch.bfloat16, heads, kv_heads, head_dim, page, segments, 61)
    for seg, row in ((0, 699), (1, 839)):
        direction = q[row, :head_dim].float()
        for place, (key, rise) in enumerate(zip((10, 130, 260, 390, 420), rises)):
            pg, off = table[seg, key // page], key % page
            k_pool[pg, 0, off] = (direction * (rise / direction.norm() ** 2 * math.sqrt(head_dim))).to(torch.bfloat16)
            v_pool[pg, 0, off] = torch.full((head_dim,), 10.0 * (place + 1)).to(torch.bfloat16)
    got, want = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    assert_close(got, want, torch.bfloat16, f"prompt attention with rising maxima {rises}")
    cuda().use_tcgen05_attention = False
    try:
        other, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
    finally:
        cuda().use_tcgen05_attention = True
    assert_close(got, other, torch.bfloat16, "tcgen05 kernel against the mma.sync kernel")


@pytest.mark.parametrize("heads,kv_heads,page,head_dim", [(2, 1, 16, 64), (6, 2, 64, 64), (4, 2, 16, 128), (2, 2, 128, 128)])
@pytest.mark.parametrize("window", [None, 333])
def test_prefill_attention_items_cut_into_parts(heads, kv_heads, page, head_dim, window):
    """Few query tiles with long key ranges: the tcgen05 kernel cuts each item's keys into up to
    eight parts that different CTAs take and the last one merges.  One far key is made dominant so
    that a part that is dropped or merged with the wrong weight shows."""
    segments = [(0, 1500), (1900, 150), (640, 1)]
    q, k_pool, v_pool, batch, table = make_attention_case(torch.bfloat16, heads, kv_heads, head_dim, page, segments, 57)
    if window is None:
        # row 1499 of the first request: key 70 dominates (its k is the scaled query of head 0)
        direction = q[1499, :head_dim].float()
        pg, off = table[0, 70 // page], 70 % page
        k_pool[pg, 0, off] = (direction * (40.0 / direction.norm() ** 2 * math.sqrt(head_dim))).to(torch.bfloat16)
        v_pool[pg, 0, off] = torch.full((head_dim,), 100.0).to(torch.bfloat16)
    got, want = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
    torch.cuda.synchronize()
    cuda().raise_if_device_error()
    assert_close(got, want, torch.bfloat16, f"prompt attention with items in parts, window={window}")
    if window is None:
        assert float(got[1499, :head_dim].float().mean()) > 90.0, "the dominant far key was lost"
    again, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
    assert torch.equal(got, again), "parts are merged in part order: same bits every time"
    cuda().split_prefill_items = False
    try:
        whole, _ = run_attention_both(torch.bfloat16, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
    finally:
        cuda().split_prefill_items = True
    assert_close(got, whole, torch.bfloat16, "items in parts against whole items")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 33, 1000])
def test_attention_window_edge(dtype, window):
    heads, kv_heads, head_dim, page = 4, 2, 32, 8
    segments = [(0, 40), (70, 3), (99, 1)]
    q, k_pool, v_pool, batch, _ = make_attention_case(dtype, heads, kv_heads, head_dim, page, segments, 22)
    got, want = run_attention_both(dtype, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, window)
    assert_close(got, want, dtype, f"attention window={window}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far_key", [0, 15, 16, 255, 256, 511, 700])
def test_attention_finds_one_far_key(dtype, far_key):
    """One key among hundreds is made to dominate (its k equals the scaled query); the output
    must then be that key's value, which no other value resembles."""
    heads, kv_heads, head_dim, page = 2, 1, 64, 16
    segments = [(700, 1), (690, 11)]
    q, k_pool, v_pool, batch, table = make_attention_case(dtype, heads, kv_heads, head_dim, page, segments, 23)
    # row 0 is the decode row at position 700; rows 1.. are the portion; take its last row (position 700)
    for seg, row in ((0, 0), (1, 11)):
        direction = q[row, :head_dim].float()
        pg, off = table[seg, far_key // page], far_key % page
        k_pool[pg, 0, off] = (direction * (40.0 / direction.norm() ** 2 * math.sqrt(head_dim))).to(dtype)
        v_pool[pg, 0, off] = torch.full((head_dim,), 100.0).to(dtype)
    got, want = run_attention_both(dtype, q, k_pool, v_pool, batch, heads, kv_heads, head_dim, None)
    assert_close(got, want, dtype, "attention with a dominant far key")
    for row in (0, 11):
        assert float(got[row, :head_dim].float().mean()) > 90.0, "the dominant key's value was lost"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_rows_do_not_depend_on_the_cut(dtype):
    """The same request as one portion, as two portions and as single rows: identical bits from
    the generic kernel (the float32 path's attention, whatever the storage type)."""
    heads, kv_heads, head_dim, page = 6, 2, 64, 16
    q, k_pool, v_pool, batch, table = make_attention_case(dtype, heads, kv_heads, head_dim, page, [(0, 45)], 24)
    scale = head_dim ** -0.5
    qd, kd, vd = q.to(DEVICE), k_pool.to(DEVICE), v_pool.to(DEVICE)
    def piece(pos0, count):
        ints = lambda v: torch.tensor(v, dtype=torch.int32, device=DEVICE)
        arrays, counts = plan_attention([count], [pos0])
        b = AttentionBatch(ints([0]), ints([count]), ints([pos0]), ints([0]), table.to(DEVICE), 1, count, pos0 + count,
                           {name: torch.from_numpy(array).to(DEVICE) for name, array in arrays.items()}, counts)
        return cuda().paged_attention(qd[pos0:pos0 + count].contiguous(), kd, vd, b, heads, kv_heads, head_dim, scale, None)

    cuda().use_mma_attention = cuda().use_decode_kernel = False      # the generic kernel for every piece
    try:
        whole = cuda().paged_attention(qd, kd, vd, batch(DEVICE), heads, kv_heads, head_dim, scale, None)
        assert torch.equal(torch.cat([piece(0, 17), piece(17, 28)]), whole)
        assert torch.equal(torch.cat([piece(p, 1) for p in range(45)]), whole)
    finally:
        cuda().use_mma_attention = cuda().use_decode_kernel = True


def test_sampling_greedy_takes_the_lowest_index_on_ties():
    logits = torch.zeros(3, 1000)
    logits[0, [17, 400, 999]] = 5.0
    logits[1, 999] = 1.0
    logits[2] = -1.0
    zeros = torch.zeros(3)
    ids = torch.zeros(3, dtype=torch.int64)
    got = cuda().sample(logits.to(DEVICE), zeros.to(DEVICE), ids.to(DEVICE), ids.to(DEVICE))
    assert got.cpu().tolist() == [17, 999, 0]


@pytest.mark.parametrize("vocab", [384, 1000, 151936])
def test_sampling_temperature_matches_the_plain_sampler(vocab):
    rows = 48
    logits = rnd((rows, vocab), torch.float32, 31, 3.0)
    temperatures = torch.linspace(0.3, 1.5, rows)
    seeds = torch.arange(rows, dtype=torch.int64) * 7919 + 11
    counters = torch.arange(rows, dtype=torch.int64) % 5
    got = cuda().sample(logits.to(DEVICE), temperatures.to(DEVICE), seeds.to(DEVICE), counters.to(DEVICE)).cpu()
    for row in range(rows):
        u = plain.uniform_from_seed(int(seeds[row]), int(counters[row]))
        token, cdf = plain.temperature_sample(logits[row], float(temperatures[row]), u)
        chosen = int(got[row])
        if chosen != token:
            # float32 summation order may move a boundary by rounding: u must then sit on it
            low = float(cdf[chosen - 1]) if chosen > 0 else 0.0
            assert low - 1e-5 <= u <= float(cdf[chosen]) + 1e-5, (row, chosen, token, u)


def test_sampling_follows_the_distribution():
    vocab, rows = 11, 4000
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0, 0.5, 3.0, -2.0, 0.0, 1.5, 2.5, -0.5]).repeat(rows, 1)
    temperatures = torch.full((rows,), 0.8)
    seeds = torch.full((rows,), 1234, dtype=torch.int64)
    counters = torch.arange(rows, dtype=torch.int64)
    got = cuda().sample(logits.to(DEVICE), temperatures.to(DEVICE), seeds.to(DEVICE), counters.to(DEVICE)).cpu()
    observed = torch.bincount(got.long(), minlength=vocab).float() / rows
    expected = torch.softmax(logits[0] / 0.8, dim=-1)
    assert float((observed - expected).abs().max()) < 0.03
