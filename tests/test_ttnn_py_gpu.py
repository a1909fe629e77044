"""The Python `ttnn` stand-in (tt-perf_b200/ttnn_py/ttnn) against torch fp32 on the CPU, op by op, with the call forms
py/engine.py, py/nn.py and py/optim.py of the reference use, plus a small autograd step assembled from them the way
the reference's engine does it (matmul + tanh forward, hand-written backward, SGD update).
Tolerance: relative Frobenius error <= 1e-2 on bf16 results."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import matmul_oracle as mo

pytestmark = pytest.mark.gpu
TOL = 1e-2
sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "tt-perf_b200" / "ttnn_py"))


@pytest.fixture(scope="module")
def tt():
    import ttnn
    dev = ttnn.open_device(device_id=0)
    yield ttnn, dev
    ttnn.close_device(dev)


def _rand(shape, seed, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).bfloat16()


def _err(got, ref):
    return mo.rel_frobenius(got.float().numpy(), ref.float().numpy())


def test_round_trip_and_attributes(tt):
    ttnn, dev = tt
    x = _rand((2, 32, 64), 1)
    t = ttnn.from_torch(x, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
    assert isinstance(t, ttnn.Tensor) and tuple(t.shape) == (2, 32, 64) and t.dtype == ttnn.bfloat16
    assert t.device() is dev and t.get_layout() == ttnn.TILE_LAYOUT
    assert torch.equal(ttnn.to_torch(t), x)
    idx = torch.randint(0, 100, (4, 32))
    ti = ttnn.from_torch(idx, device=dev, layout=ttnn.ROW_MAJOR_LAYOUT, dtype=ttnn.uint32)
    assert ti.dtype == ttnn.uint32 and torch.equal(ttnn.to_torch(ti).long(), idx)
    with pytest.raises(NotImplementedError):
        ttnn.from_torch(x.float(), device=dev, dtype=ttnn.float32)


def test_binary_broadcast_scalar_and_unary_ops(tt):
    ttnn, dev = tt
    a, b = _rand((2, 4, 32, 64), 2), _rand((1, 1, 32, 64), 3)
    row, col = _rand((2, 4, 32, 1), 4), _rand((64,), 5)
    ta, tb, tr, tc = (ttnn.from_torch(v, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16) for v in (a, b, row, col))
    af, bf, rf, cf = a.float(), b.float(), row.float(), col.float()
    assert _err(ttnn.to_torch(ttnn.add(ta, tb)), af + bf) <= TOL
    assert _err(ttnn.to_torch(ttnn.sub(ta, tr)), af - rf) <= TOL
    assert _err(ttnn.to_torch(ttnn.mul(ta, tc)), af * cf) <= TOL
    assert _err(ttnn.to_torch(ttnn.div(ta, ttnn.full_like(ta, fill_value=3.0))), af / 3.0) <= TOL
    assert _err(ttnn.to_torch(ttnn.mul(ta, 0.5)), af * 0.5) <= TOL
    assert _err(ttnn.to_torch(ttnn.tanh(ta)), torch.tanh(af)) <= TOL
    assert _err(ttnn.to_torch(ttnn.relu(ta)), torch.relu(af)) <= TOL
    assert torch.equal(ttnn.to_torch(ttnn.gtz(ta)).float(), (af > 0).float())
    pos = ttnn.add(ttnn.mul(ta, ta), 1.0)
    pf = (af * af).bfloat16().float() + 1.0
    assert _err(ttnn.to_torch(ttnn.sqrt(pos)), torch.sqrt(pf)) <= TOL
    assert _err(ttnn.to_torch(ttnn.log(pos)), torch.log(pf)) <= TOL
    assert _err(ttnn.to_torch(ttnn.exp(ttnn.mul(ta, 0.1))), torch.exp((af * 0.1).bfloat16().float())) <= TOL
    assert torch.equal(ttnn.to_torch(ttnn.ones_like(ta)).float(), torch.ones_like(af))


def test_matmul_forms_of_the_engine(tt):
    ttnn, dev = tt
    x, w = _rand((2, 64, 96), 6), _rand((96, 128), 7, 0.1)
    g = _rand((2, 64, 128), 8)
    tx, tw, tg = (ttnn.from_torch(v, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16) for v in (x, w, g))
    y = ttnn.matmul(tx, tw)                                       # forward  [B,S,K] x [K,N]
    assert tuple(y.shape) == (2, 64, 128) and _err(ttnn.to_torch(y), x.float() @ w.float()) <= TOL
    gx = ttnn.matmul(tg, tw, transpose_b=True)                    # grad_self = g . w^T      (py/engine.py:298)
    assert _err(ttnn.to_torch(gx), g.float() @ w.float().T) <= TOL
    gw = ttnn.matmul(tx, tg, transpose_a=True)                    # grad_other = x^T . g, per batch (py/engine.py:304)
    assert tuple(gw.shape) == (2, 96, 128)
    assert _err(ttnn.to_torch(gw), x.float().transpose(1, 2) @ g.float()) <= TOL
    gw0 = ttnn.sum(gw, dim=0, keepdim=False)                      # _reduce_to_shape over the broadcast batch
    assert _err(ttnn.to_torch(gw0), (x.float().transpose(1, 2) @ g.float()).sum(0)) <= TOL
    q, k = _rand((2, 3, 64, 32), 9), _rand((2, 3, 64, 32), 10)
    tq, tk = (ttnn.from_torch(v, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16) for v in (q, k))
    s = ttnn.matmul(tq, tk, transpose_b=True, compute_kernel_config=ttnn.WormholeComputeKernelConfig(
        math_fidelity=ttnn.MathFidelity.HiFi3))
    assert _err(ttnn.to_torch(s), q.float() @ k.float().transpose(-1, -2)) <= TOL


def test_softmax_logsoftmax_cross_entropy_chain(tt):
    """The op chain of py/nn.py:170-218: softmax, log, one-hot product, sums, and the gradient (p - onehot) * scale."""
    ttnn, dev = tt
    batch, seq, classes = 2, 32, 96
    logits = _rand((batch, seq, classes), 11, 2.0)
    targets = torch.randint(0, classes, (batch * seq,), generator=torch.Generator().manual_seed(12))
    tl = ttnn.from_torch(logits, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
    flat = ttnn.reshape(tl, (batch * seq, classes))
    one_hot = torch.nn.functional.one_hot(targets, classes).bfloat16()
    toh = ttnn.from_torch(one_hot, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
    p = ttnn.softmax(flat, dim=-1)
    logp = ttnn.log(p)
    nll = ttnn.sum(ttnn.mul(toh, logp), dim=-1, keepdim=False)
    nll = ttnn.mul(nll, ttnn.full_like(nll, fill_value=-1.0))
    total = ttnn.sum(nll, dim=0, keepdim=False)
    loss = ttnn.mul(total, ttnn.full_like(total, fill_value=1.0 / (batch * seq)))
    ref = torch.nn.functional.cross_entropy(logits.float().reshape(-1, classes), targets)
    assert abs(ttnn.to_torch(loss).float().item() - ref.item()) <= 1e-2 * abs(ref.item())
    grad = ttnn.mul(ttnn.sub(p, toh), ttnn.full_like(p, fill_value=1.0 / (batch * seq)))
    ref_p = torch.softmax(logits.float().reshape(-1, classes), -1)
    assert _err(ttnn.to_torch(grad), (ref_p - one_hot.float()) / (batch * seq)) <= TOL
    # softmax backward of the engine (py/engine.py:361-362) and a softmax over a middle dimension
    dy = _rand((batch * seq, classes), 13)
    tdy = ttnn.from_torch(dy, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
    dot = ttnn.sum(ttnn.mul(tdy, p), dim=-1, keepdim=True)
    gin = ttnn.mul(p, ttnn.sub(tdy, dot))
    assert _err(ttnn.to_torch(gin), ref_p * (dy.float() - (dy.float() * ref_p).sum(-1, keepdim=True))) <= 1e-2
    mid = ttnn.softmax(tl, dim=1)
    assert _err(ttnn.to_torch(mid), torch.softmax(logits.float(), 1)) <= TOL


def test_layout_ops_mask_and_embedding(tt):
    ttnn, dev = tt
    x = _rand((2, 32, 4, 16), 14)
    tx = ttnn.from_torch(x, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
    assert torch.equal(ttnn.to_torch(ttnn.permute(tx, (0, 2, 1, 3))), x.permute(0, 2, 1, 3).contiguous())
    assert torch.equal(ttnn.to_torch(ttnn.reshape(tx, (2, 32, 64))), x.reshape(2, 32, 64))
    s = ttnn.from_torch(_rand((3, 32, 32), 15), device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
    mask = ttnn.triu(ttnn.full_like(s, fill_value=-1e9), diagonal=1)             # py/nn.py:248-249
    ref_mask = torch.triu(torch.full((3, 32, 32), -1e9), diagonal=1).bfloat16()
    assert torch.equal(ttnn.to_torch(mask), ref_mask)
    table = _rand((50, 64), 16)
    idx = torch.randint(0, 50, (2, 32), generator=torch.Generator().manual_seed(17))
    tt_idx = ttnn.from_torch(idx, device=dev, layout=ttnn.ROW_MAJOR_LAYOUT, dtype=ttnn.uint32)
    tt_idx = ttnn.reshape(tt_idx, (64,))
    emb = ttnn.embedding(tt_idx, ttnn.from_torch(table, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16),
                         layout=ttnn.TILE_LAYOUT)
    assert torch.equal(ttnn.to_torch(ttnn.reshape(emb, (2, 32, 64))), table[idx])
    red = ttnn.from_torch(_rand((4, 32, 64), 18), device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
    assert _err(ttnn.to_torch(ttnn.sum(red, dim=1, keepdim=True)), ttnn.to_torch(red).float().sum(1, keepdim=True)) <= TOL


def test_tanh_layer_backward_and_sgd_like_the_engine(tt):
    """y = tanh(x w); loss gradient g; dW = x^T (g * (1 - y^2)); w <- w - lr * dW, in the engine's op sequence
    (py/engine.py:314-322, :298-307; py/optim.py:19-21)."""
    ttnn, dev = tt
    x, w, g = _rand((64, 96), 19), _rand((96, 32), 20, 0.2), _rand((64, 32), 21)
    tx, tw, tg = (ttnn.from_torch(v, device=dev, layout=ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16) for v in (x, w, g))
    y = ttnn.tanh(ttnn.matmul(tx, tw))
    dy = ttnn.mul(ttnn.sub(ttnn.ones_like(y), ttnn.mul(y, y)), tg)
    dw = ttnn.matmul(tx, dy, transpose_a=True)
    new_w = ttnn.sub(tw, ttnn.mul(dw, ttnn.full_like(dw, fill_value=0.1)))
    xf, wf, gf = x.float(), w.float(), g.float()
    yf = torch.tanh(xf @ wf)
    ref = wf - 0.1 * (xf.T @ ((1 - yf * yf) * gf))
    assert _err(ttnn.to_torch(new_w), ref) <= TOL
