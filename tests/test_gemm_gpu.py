"""Parity of b200_gemm (called through the C ABI) with the CPU oracle: relative Frobenius error <= 1e-2 for
bf16 outputs (the tolerance the hot path is specified to), on seeded inputs, for the three product forms the
executors use — forward x.W^T (NT), dX = dY.W (NN), dW = dY^T.X (TN) — over aligned, ragged, tiny, batched,
split-K and fused-epilogue cases."""
import json

import numpy as np
import pytest
import torch

from oracle import matmul_oracle as mo
from conftest import GOLDEN

pytestmark = pytest.mark.gpu
TOL = 1e-2


def dev_bf16(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).bfloat16().cuda()


def run_gemm(pkg, ctx, stream, a, b, M, N, K, *, ta=False, tb=False, batch=1, c_dtype=None, poison=True, **kw):
    c_dtype = pkg.BF16 if c_dtype is None else c_dtype
    tdt = torch.bfloat16 if c_dtype == pkg.BF16 else torch.float32
    shape = (batch, M, N) if batch > 1 else (M, N)
    c = torch.full(shape, float("nan"), dtype=tdt, device="cuda") if poison else torch.empty(shape, dtype=tdt, device="cuda")
    ctx.gemm(ctx.gemm_desc(a, b, c, M, N, K, transpose_a=ta, transpose_b=tb, batch=batch, c_dtype=c_dtype, **kw),
             stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    return c


def operands(M, N, K, ta, tb, batch=1, seed=0, scale=1.0):
    rng = np.random.default_rng(seed + 1000003 * M + 1009 * N + K)
    a_shape = (K, M) if ta else (M, K)
    b_shape = (N, K) if tb else (K, N)
    if batch > 1:
        a_shape, b_shape = (batch,) + a_shape, (batch,) + b_shape
    a = mo.bf16_round(rng.standard_normal(a_shape).astype(np.float32) * scale)
    b = mo.bf16_round(rng.standard_normal(b_shape).astype(np.float32) * scale)
    return a, b


FORMS = [(False, True), (False, False), (True, False), (True, True)]
SHAPES = [
    (32, 32, 64),       # the KAT size of autograd/tests/test_matmul.cpp
    (128, 256, 64),     # exactly one tile, one K block
    (128, 256, 512),
    (256, 512, 512),
    (200, 264, 136),    # ragged in every dimension
    (1000, 520, 776),
    (64, 128, 784),     # MLP layer 1 (K = 784)
    (1024, 512, 512),   # the bench_autograd layer
    (8, 8, 8),
    (1, 8, 8),
    (513, 72, 1032),
    (2600, 2824, 776),  # enough 256 x 256 tiles for the CTA-pair kernel, ragged on every side
    (4096, 2560, 320),
]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("ta,tb", FORMS)
@pytest.mark.parametrize("algo", ["tcgen05", "simt"])
def test_gemm_matches_oracle(pkg, ctx, stream, M, N, K, ta, tb, algo):
    lda = M if ta else K
    ldb = K if tb else N
    if algo == "tcgen05" and (lda % 8 or ldb % 8):
        pytest.skip("TMA path needs 16-byte aligned rows; covered by the SIMT case and the AUTO test")
    a, b = operands(M, N, K, ta, tb)
    c = run_gemm(pkg, ctx, stream, dev_bf16(a), dev_bf16(b), M, N, K, ta=ta, tb=tb,
                 algo=pkg.ALGO_TCGEN05 if algo == "tcgen05" else pkg.ALGO_SIMT)
    got = c.float().cpu().numpy()
    assert not np.isnan(got).any(), "output tile left unwritten"
    assert mo.rel_frobenius(got, mo.matmul(a, b, ta, tb)) <= TOL


def test_known_answer_ones(pkg, ctx, stream):
    """autograd/tests/test_matmul.cpp:17-34 / verify/verify_autograd.py: ones[32,64].ones[64,32] = 64, dA = dB = 32;
    exact in bf16."""
    gold = json.loads((GOLDEN / "verify_autograd.json").read_text())["matmul"]
    a = torch.ones(32, 64, dtype=torch.bfloat16, device="cuda")
    b = torch.ones(64, 32, dtype=torch.bfloat16, device="cuda")
    d_c = torch.ones(32, 32, dtype=torch.bfloat16, device="cuda")
    c = run_gemm(pkg, ctx, stream, a, b, 32, 32, 64)
    d_a = run_gemm(pkg, ctx, stream, d_c, b, 32, 64, 32, tb=True)      # dA = dC . B^T
    d_b = run_gemm(pkg, ctx, stream, a, d_c, 64, 32, 32, ta=True)      # dB = A^T . dC
    assert torch.all(c.float() == gold["C"]) and torch.all(d_a.float() == gold["dA"]) and torch.all(d_b.float() == gold["dB"])


def test_unaligned_shapes_take_the_simt_path_automatically(pkg, ctx, stream):
    """[64,10] logits of the 784-128-10 MLP: rows of 20 bytes cannot be TMA sources, AUTO must still work."""
    for (M, N, K, ta, tb) in [(64, 10, 128, False, True), (64, 128, 10, False, False), (10, 128, 64, True, False)]:
        a, b = operands(M, N, K, ta, tb, seed=5)
        c = run_gemm(pkg, ctx, stream, dev_bf16(a), dev_bf16(b), M, N, K, ta=ta, tb=tb)
        assert mo.rel_frobenius(c.float().cpu().numpy(), mo.matmul(a, b, ta, tb)) <= TOL
    a, b = operands(64, 10, 128, False, True)
    with pytest.raises(pkg.B200Error) as e:
        run_gemm(pkg, ctx, stream, dev_bf16(a)[:, 1:], dev_bf16(b), 64, 10, 127, tb=True, lda=128,
                 algo=pkg.ALGO_TCGEN05)
    assert e.value.code == pkg.capi.ERR_INVALID_ARG


@pytest.mark.parametrize("ta,tb", FORMS[:3])
def test_batched_and_broadcast(pkg, ctx, stream, ta, tb):
    """[B,H,S,dh] attention products (traced/nn.hpp:166-191) and a rank-2 weight broadcast over the batch
    (traced/transformer.hpp:198)."""
    batch, M, N, K = 6, 96, 64, 160
    a, b = operands(M, N, K, ta, tb, batch=batch, seed=9)
    c = run_gemm(pkg, ctx, stream, dev_bf16(a), dev_bf16(b), M, N, K, ta=ta, tb=tb, batch=batch)
    assert mo.rel_frobenius(c.float().cpu().numpy(), mo.matmul(a, b, ta, tb)) <= TOL
    c = run_gemm(pkg, ctx, stream, dev_bf16(a), dev_bf16(b[0]), M, N, K, ta=ta, tb=tb, batch=batch, stride_b=0)
    assert mo.rel_frobenius(c.float().cpu().numpy(), mo.matmul(a, b[0], ta, tb)) <= TOL


@pytest.mark.parametrize("split", [0, 2, 3, 7])
@pytest.mark.parametrize("ta,tb", FORMS[:3])
def test_split_k(pkg, ctx, stream, split, ta, tb):
    """dW = dY^T . X reduces over all tokens (K large, M and N small): K is cut into slices whose fp32 partial
    sums go through scratch memory and a reduce kernel."""
    M, N, K = 264, 200, 2056
    a, b = operands(M, N, K, ta, tb, seed=21)
    bias = mo.bf16_round(np.random.default_rng(2).standard_normal(N).astype(np.float32))
    d = ctx.gemm_desc(None, None, None, M, N, K, transpose_a=ta, transpose_b=tb, split_k=split)
    c = run_gemm(pkg, ctx, stream, dev_bf16(a), dev_bf16(b), M, N, K, ta=ta, tb=tb, split_k=split,
                 bias=dev_bf16(bias), activation=pkg.ACT_RELU, algo=pkg.ALGO_TCGEN05)
    ref = mo.relu(mo.matmul(a, b, ta, tb) + bias)
    assert mo.rel_frobenius(c.float().cpu().numpy(), ref) <= TOL
    if split > 1:
        assert d.split_k == split


def test_split_k_scratch_query(pkg, ctx):
    d = ctx.gemm_desc(0x1000, 0x1000, 0x1000, 768, 768, 8192, transpose_a=True)
    n = ctx.gemm_scratch_bytes(d)
    assert n > 0 and n % (768 * 768 * 4) == 0
    d = ctx.gemm_desc(0x1000, 0x1000, 0x1000, 8192, 8192, 8192)
    assert ctx.gemm_scratch_bytes(d) == 0


@pytest.mark.parametrize("algo", ["tcgen05", "simt"])
def test_fused_epilogues(pkg, ctx, stream, algo):
    """ttnn::linear(x, w, bias, ..., "relu") (static/nn.hpp:145-146), GELU, alpha scaling with the causal mask
    (traced/nn.hpp:166-168), fp32 output (fp32_dest_acc_en, verify/verify_fidelity.cpp:50-55)."""
    algo_id = pkg.ALGO_TCGEN05 if algo == "tcgen05" else pkg.ALGO_SIMT
    M, N, K = 160, 328, 264
    a, b = operands(M, N, K, False, True, seed=3, scale=0.5)
    bias = mo.bf16_round(np.random.default_rng(4).standard_normal(N).astype(np.float32))
    da, db, dbias = dev_bf16(a), dev_bf16(b), dev_bf16(bias)
    base = mo.matmul(a, b, False, True)
    c = run_gemm(pkg, ctx, stream, da, db, M, N, K, tb=True, bias=dbias, algo=algo_id)
    assert mo.rel_frobenius(c.float().cpu().numpy(), base + bias) <= TOL
    c = run_gemm(pkg, ctx, stream, da, db, M, N, K, tb=True, bias=dbias, activation=pkg.ACT_RELU, algo=algo_id)
    assert mo.rel_frobenius(c.float().cpu().numpy(), mo.linear_forward(a, b, bias, "relu")) <= TOL
    c = run_gemm(pkg, ctx, stream, da, db, M, N, K, tb=True, bias=dbias, activation=pkg.ACT_GELU, algo=algo_id)
    assert mo.rel_frobenius(c.float().cpu().numpy(), mo.linear_forward(a, b, bias, "gelu")) <= TOL
    c = run_gemm(pkg, ctx, stream, da, db, M, N, K, tb=True, bias=torch.from_numpy(bias).cuda(),
                 bias_dtype=pkg.F32, c_dtype=pkg.F32, algo=algo_id)
    assert c.dtype == torch.float32 and mo.rel_frobenius(c.cpu().numpy(), base + bias) <= 1e-5
    # scale + causal mask, square scores
    S, dh = 192, 64
    q, k = operands(S, S, dh, False, True, seed=8)
    c = run_gemm(pkg, ctx, stream, dev_bf16(q), dev_bf16(k), S, S, dh, tb=True, alpha=0.125, causal_mask=True,
                 mask_value=-1e9, c_dtype=pkg.F32, algo=algo_id)
    ref = mo.matmul(q, k, False, True) * np.float32(0.125)
    got = c.cpu().numpy()
    low = np.tril(np.ones((S, S), bool))
    assert mo.rel_frobenius(got[low], ref[low]) <= 1e-5 and np.all(got[~low] == np.float32(-1e9))


def test_fidelity_levels_stay_within_tolerance(pkg, ctx, stream):
    """verify/verify_fidelity.cpp:50-55: LoFi / HiFi2 / HiFi3 / HiFi4 — here they select the precision of the
    split-K partial sums and the GELU form; all must stay inside the parity tolerance."""
    M, N, K = 256, 256, 4096
    a, b = operands(M, N, K, True, False, seed=13, scale=0.25)
    ref = mo.gelu(mo.matmul(a, b, True, False))
    outs = []
    for fid in (pkg.LOFI, pkg.HIFI2, pkg.HIFI3, pkg.HIFI4):
        c = run_gemm(pkg, ctx, stream, dev_bf16(a), dev_bf16(b), M, N, K, ta=True, fidelity=fid, split_k=4,
                     activation=pkg.ACT_GELU, algo=pkg.ALGO_TCGEN05)
        outs.append(c.float().cpu().numpy())
        assert mo.rel_frobenius(outs[-1], ref) <= TOL
    assert np.array_equal(outs[2], outs[3])


def test_empty_and_degenerate_products(pkg, ctx, stream):
    a = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    c = torch.full((8, 8), 7.0, dtype=torch.bfloat16, device="cuda")
    s = stream.cuda_stream
    ctx.gemm(ctx.gemm_desc(a, a, c, 0, 8, 8), s)        # M = 0: nothing written
    ctx.gemm(ctx.gemm_desc(a, a, c, 8, 0, 8, ldc=8), s)  # N = 0
    ctx.synchronize(s)
    assert torch.all(c == 7.0)
    bias = torch.arange(8, dtype=torch.float32).bfloat16().cuda()
    ctx.gemm(ctx.gemm_desc(a, a, c, 8, 8, 0, lda=8, ldb=8, bias=bias), s)  # K = 0: C = bias
    ctx.synchronize(s)
    assert torch.all(c.float() == bias.float()[None, :])
    for bad in (dict(M=-1), dict(batch=0), dict(ldc=4), dict(c_dtype=7), dict(activation=9)):
        kw = dict(M=8, N=8, K=8)
        kw.update({k: v for k, v in bad.items() if k in ("M",)})
        d = ctx.gemm_desc(a, a, c, kw["M"], 8, 8)
        for k, v in bad.items():
            setattr(d, k, v)
        with pytest.raises(pkg.B200Error) as e:
            ctx.gemm(d, s)
        assert e.value.code == pkg.capi.ERR_INVALID_ARG


def test_run_twice_bitwise_identical(pkg, ctx, stream):
    """Races on the mbarrier / TMEM hand-offs would show up as run-to-run differences."""
    M, N, K = 1024, 1024, 1024
    a, b = operands(M, N, K, False, False, seed=77)
    da, db = dev_bf16(a), dev_bf16(b)
    outs = [run_gemm(pkg, ctx, stream, da, db, M, N, K, algo=pkg.ALGO_TCGEN05).clone() for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


@pytest.mark.parametrize("ta,tb", FORMS[:3])
def test_full_size_8192_linearity_and_row_sample(pkg, ctx, stream, ta, tb):
    """Full benchmark size: a sample of output rows against the oracle, plus a size-independent property —
    the product is linear in A, so (A1 + A2).B == A1.B + A2.B up to bf16 rounding of the three outputs."""
    M = N = K = 8192
    g = torch.Generator(device="cuda").manual_seed(42)
    a1 = torch.randn((K, M) if ta else (M, K), generator=g, device="cuda").bfloat16()
    b = torch.randn((N, K) if tb else (K, N), generator=g, device="cuda").bfloat16()
    c1 = run_gemm(pkg, ctx, stream, a1, b, M, N, K, ta=ta, tb=tb, poison=False)
    rows = np.arange(0, M, 1171)
    a_rows = (a1[:, rows].t() if ta else a1[rows]).float().cpu().numpy()
    b_np = b.float().cpu().numpy()
    ref = mo.matmul(a_rows, b_np, False, tb)
    assert mo.rel_frobenius(c1[rows].float().cpu().numpy(), ref) <= TOL
    a2 = a1.flip(0).contiguous()          # exactly representable second operand
    a_sum = (a1.float() + a2.float())     # may round when stored as bf16: use 2*a1 instead for exactness
    del a_sum
    c2 = run_gemm(pkg, ctx, stream, (a1.float() * 2).bfloat16(), b, M, N, K, ta=ta, tb=tb, poison=False)
    # scaling A by 2 is exact in bf16, so the product must be exactly doubled
    assert torch.equal(c2.float(), c1.float() * 2)
    del a2


@pytest.mark.parametrize("M,N,K,stride", [(16384, 16384, 16384, 1489), (128, 8192, 8192, 1), (4096, 4096, 4096, 257),
                                            (2048, 2048, 2048, 129), (1024, 1024, 1024, 65), (512, 512, 512, 33)])
def test_sweep_shapes_row_sample(pkg, ctx, stream, M, N, K, stride):
    """The other shapes of the matmul sweep (512^3 .. 16384^3 and the skinny M = 128, K = N = 8192 product, which the
    planner cuts along K): seeded N(0,1) operands, a sample of output rows against the oracle, and exact doubling."""
    g = torch.Generator(device="cuda").manual_seed(42)
    a = torch.randn((M, K), generator=g, device="cuda").bfloat16()
    b = torch.randn((K, N), generator=g, device="cuda").bfloat16()
    c = run_gemm(pkg, ctx, stream, a, b, M, N, K)
    assert not torch.isnan(c).any(), "output tile left unwritten"
    rows = np.arange(0, M, stride)
    ref = mo.matmul(a[rows].float().cpu().numpy(), b.float().cpu().numpy())
    assert mo.rel_frobenius(c[rows].float().cpu().numpy(), ref) <= TOL
    c2 = run_gemm(pkg, ctx, stream, (a.float() * 2).bfloat16(), b, M, N, K, poison=False)
    assert torch.equal(c2.float(), c.float() * 2)


@pytest.mark.parametrize("M,N,K,ta,tb", [(1024, 512, 384, False, False), (1000, 520, 776, False, True),
                                          (2048, 264, 512, True, False), (300, 72, 40, False, False)])
def test_matmul_host_buffers_pipelined(pkg, ctx, M, N, K, ta, tb):
    """b200_matmul_host: operands and result in host memory (pinned or pageable), upload / compute / download
    pipelined over row panels — the from_vector -> to_device -> matmul -> cpu() path of a reference program."""
    a, b = operands(M, N, K, ta, tb, seed=31)
    a_h = torch.from_numpy(a).bfloat16().pin_memory()
    b_h = torch.from_numpy(b).bfloat16()                     # pageable on purpose
    c_h = torch.full((M, N), float("nan"), dtype=torch.bfloat16).pin_memory()
    d = ctx.gemm_desc(a_h, b_h, c_h, M, N, K, transpose_a=ta, transpose_b=tb)
    for panels in (0, 3):
        c_h.fill_(float("nan"))
        ctx.matmul_host(d, panels)
        got = c_h.float().numpy()
        assert not np.isnan(got).any()
        assert mo.rel_frobenius(got, mo.matmul(a, b, ta, tb)) <= TOL
