"""Host-side mirror of the reference's layer vocabulary over the C ABI: Linear, ReLU/GELU, causal attention,
LayerNorm, cross-entropy, SGD/Adam, the 2-layer MLP train step and the pre-LN GPT-2 block forward/backward.

Every function only sequences C-ABI calls on device tensors (tt-perf_b200/tensor.py); no arithmetic happens on
the host. Names and argument meaning follow the reference's traced executor: `linear_forward/backward`
(autograd/traced/ops.hpp:113-119, traced/nn.hpp:72-90), `TracedCausalAttention` (traced/nn.hpp:164-192),
`TracedLayerNorm` (traced/nn.hpp:226-269), `TracedMLP::train_step` (traced/mlp.hpp:72-117), the trainable
transformer layer (traced/transformer_train.hpp:179-257) with the gradient forms corrected as in
verify/compare_grads.py:234-249 (weights' gradients reduce over batch AND sequence)."""
from __future__ import annotations

import math

import numpy as np

from . import capi
from .capi import ACT_GELU, ACT_NONE, ACT_RELU, BF16, F32, FP8_E4M3
from .tensor import DeviceTensor

_ACT = {None: ACT_NONE, "relu": ACT_RELU, "gelu": ACT_GELU}


def _rows(t: DeviceTensor) -> int:
    return t.numel // t.shape[-1]


def matmul(ctx, a: DeviceTensor, b: DeviceTensor, transpose_a=False, transpose_b=False, *, stream=None, alpha=1.0,
           causal_mask=False, bias=None, activation=None, out_dtype=BF16, **kw) -> DeviceTensor:
    """ttnn::matmul(a, b, transpose_a, transpose_b) with leading dims batched; a rank-2 `b` broadcasts."""
    am, ak = (a.shape[-1], a.shape[-2]) if transpose_a else (a.shape[-2], a.shape[-1])
    bk, bn = (b.shape[-1], b.shape[-2]) if transpose_b else (b.shape[-2], b.shape[-1])
    if ak != bk:
        raise ValueError(f"matmul: inner dimensions differ ({a.shape} x {b.shape}, ta={transpose_a}, tb={transpose_b})")
    lead_a, lead_b = a.shape[:-2], b.shape[:-2]
    batch = int(math.prod(lead_a)) if lead_a else 1
    if len(b.shape) == 2:
        if transpose_a and batch > 1:
            raise ValueError("matmul: a transposed batched lhs needs a batched rhs")
        # [B.., M, K] x [K, N]: fold the batch into M (one big GEMM)
        m_total = batch * am if not transpose_a else am
        out = DeviceTensor(ctx, lead_a + (am, bn), out_dtype)
        d = ctx.gemm_desc(a, b, out, m_total, bn, ak, transpose_a=transpose_a, transpose_b=transpose_b, alpha=alpha,
                          causal_mask=causal_mask, bias=bias, activation=_ACT[activation], c_dtype=out_dtype, **kw)
    else:
        if lead_a != lead_b:
            raise ValueError(f"matmul: batch dims differ ({a.shape} x {b.shape})")
        out = DeviceTensor(ctx, lead_a + (am, bn), out_dtype)
        d = ctx.gemm_desc(a, b, out, am, bn, ak, transpose_a=transpose_a, transpose_b=transpose_b, batch=batch, alpha=alpha,
                          causal_mask=causal_mask, bias=bias, activation=_ACT[activation], c_dtype=out_dtype, **kw)
    ctx.gemm(d, stream)
    return out


def linear_forward(ctx, x, w, bias=None, activation=None, *, stream=None) -> DeviceTensor:
    """y = act(x . w^T + b); w is [out, in] (ttnn::linear(x, w, bias, false, true, ..., "relu"))."""
    return matmul(ctx, x, w, False, True, bias=bias, activation=activation, stream=stream)


E4M3_MAX = 448.0


def quantize_fp8(ctx, x: DeviceTensor, *, scale=None, transposed=False, stream=None):
    """Returns (codes, scale): codes = e4m3(x * scale) as a one-byte-per-element tensor of x's shape, or of the
    transposed shape [cols, rows] of x viewed as a matrix over its last dimension (transposed=True: the copy a
    dX or dW product reads, since 8-bit operands are K-major only).
    scale=None picks 448 / max|x| (one reduction and a host read of its result, so not for use while a trace is
    being recorded); a caller that tracks the range itself passes its scale and stays asynchronous."""
    if scale is None:
        amax = DeviceTensor(ctx, (1,), F32)
        ctx.absmax(x, x.numel, amax, stream=stream)
        peak = float(amax.numpy(stream)[0])
        scale = E4M3_MAX / peak if peak > 0.0 else 1.0
    if transposed:
        rows, cols = _rows(x), x.shape[-1]
        q = DeviceTensor(ctx, (cols, rows), FP8_E4M3)
        ctx.quantize_fp8_transposed(x, rows, cols, scale, q, stream=stream)
    else:
        q = DeviceTensor(ctx, x.shape, FP8_E4M3)
        ctx.quantize_fp8(x, x.numel, scale, q, stream=stream)
    return q, float(scale)


def linear_forward_fp8(ctx, x_q, x_scale, w_q, w_scale, bias=None, activation=None, *, out_dtype=BF16, stream=None):
    """y = act((x_q . w_q^T) / (x_scale * w_scale) + b) on 8-bit operands at twice the bf16 tensor rate; x_q [.., in] and
    w_q [out, in] come from quantize_fp8. The reduced-precision Linear of the fidelity study
    (verify/verify_fidelity.cpp:151-208) on this hardware's low-precision operand format."""
    return matmul(ctx, x_q, w_q, False, True, bias=bias, activation=activation, out_dtype=out_dtype, stream=stream,
                  alpha=1.0 / (x_scale * w_scale), ab_dtype=FP8_E4M3)


def linear_backward(ctx, x, w, d_y, *, need_dx=True, need_db=True, stream=None):
    """Returns (dx, dW, db): dx = dy . w, dW = dy^T . x and db = column sums of dy over all leading positions."""
    rows, n_out, n_in = _rows(x), w.shape[0], w.shape[1]
    x2, dy2 = x.reshape(rows, n_in), d_y.reshape(rows, n_out)
    d_x = matmul(ctx, d_y, w, False, False, stream=stream) if need_dx else None
    d_w = matmul(ctx, dy2, x2, True, False, stream=stream)
    d_b = None
    if need_db:
        d_b = DeviceTensor(ctx, (n_out,), BF16)
        ctx.reduce(capi.R_SUM, dy2, 1, rows, n_out, d_b, stream=stream)
    return d_x, d_w, d_b


def relu_backward(ctx, d_y, x_pre, *, stream=None) -> DeviceTensor:
    out = DeviceTensor(ctx, d_y.shape, BF16)
    ctx.binary(capi.B_RELU_BW, d_y, (d_y.numel,), x_pre, (x_pre.numel,), out, stream=stream)
    return out


def gelu_backward(ctx, d_y, x_pre, *, want_colsum=False, stream=None):
    """dx = dy * GELU'(x_pre). want_colsum also returns the column sums of dx over all leading positions (bf16 [cols]):
    dx is the dY of the Linear layer in front of the GELU, so they are that layer's bias gradient, from the same pass."""
    out = DeviceTensor(ctx, d_y.shape, BF16)
    if not want_colsum:
        ctx.binary(capi.B_GELU_BW, d_y, (d_y.numel,), x_pre, (x_pre.numel,), out, stream=stream)
        return out
    cols = d_y.shape[-1]
    colsum = DeviceTensor(ctx, (cols,), BF16)
    ctx.gelu_backward(d_y, x_pre, out, colsum, _rows(d_y), cols, stream=stream)
    return out, colsum


def add(ctx, a, b, *, stream=None) -> DeviceTensor:
    out = DeviceTensor(ctx, a.shape, BF16)
    ctx.binary(capi.B_ADD, a, a.shape, b, b.shape, out, stream=stream)
    return out


def layernorm_forward(ctx, x, gamma, beta, *, eps=1e-5, stream=None):
    rows, cols = _rows(x), x.shape[-1]
    y = DeviceTensor(ctx, x.shape, BF16)
    mean, rstd = DeviceTensor(ctx, (rows,), F32), DeviceTensor(ctx, (rows,), F32)
    ctx.layernorm_forward(x, gamma, beta, y, mean, rstd, rows, cols, eps=eps, stream=stream)
    return y, mean, rstd


def add_layernorm_forward(ctx, x, residual, gamma, beta, *, eps=1e-5, stream=None):
    """(x + residual, LayerNorm(x + residual), mean, rstd) in one pass over the rows."""
    rows, cols = _rows(x), x.shape[-1]
    total, y = DeviceTensor(ctx, x.shape, BF16), DeviceTensor(ctx, x.shape, BF16)
    mean, rstd = DeviceTensor(ctx, (rows,), F32), DeviceTensor(ctx, (rows,), F32)
    ctx.add_layernorm_forward(x, residual, total, gamma, beta, y, mean, rstd, rows, cols, eps=eps, stream=stream)
    return total, y, mean, rstd


def layernorm_backward(ctx, d_y, x, gamma, mean, rstd, *, upstream=None, want_colsum=False, stream=None):
    """(dx, dgamma, dbeta); with `upstream`, dx also includes that gradient (the residual path) without a separate add.
    want_colsum appends the column sums of dx (bf16 [cols]): dx is the dY of the Linear layer that writes into this
    residual stream, so the sums are that layer's bias gradient."""
    rows, cols = _rows(x), x.shape[-1]
    d_x = DeviceTensor(ctx, x.shape, BF16)
    dg, db = DeviceTensor(ctx, (cols,), F32), DeviceTensor(ctx, (cols,), F32)
    if want_colsum:
        cs = DeviceTensor(ctx, (cols,), BF16)
        ctx.layernorm_backward_full(d_y, x, gamma, mean, rstd, upstream, d_x, dg, db, cs, rows, cols, stream=stream)
        return d_x, dg, db, cs
    if upstream is None:
        ctx.layernorm_backward(d_y, x, gamma, mean, rstd, d_x, dg, db, rows, cols, stream=stream)
    else:
        ctx.layernorm_backward_add(d_y, x, gamma, mean, rstd, upstream, d_x, dg, db, rows, cols, stream=stream)
    return d_x, dg, db


def causal_attention_forward(ctx, q, k, v, *, scale=None, stream=None):
    """q, k, v: [..., S, dh]. scores = q k^T with the 1/sqrt(dh) scale and the causal mask fused into one softmax
    pass; returns (O, P) with P kept for the backward pass."""
    s_len, dh = q.shape[-2], q.shape[-1]
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    scores = matmul(ctx, q, k, False, True, stream=stream)
    p = DeviceTensor(ctx, scores.shape, BF16)
    ctx.softmax(scores, p, _rows(scores), s_len, alpha=scale, causal_period=s_len, stream=stream)
    return matmul(ctx, p, v, stream=stream), p


def causal_attention_backward(ctx, q, k, v, p, d_o, *, scale=None, stream=None):
    dh = q.shape[-1]
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    d_v = matmul(ctx, p, d_o, True, False, stream=stream)
    d_p = matmul(ctx, d_o, v, False, True, stream=stream)
    d_s = DeviceTensor(ctx, p.shape, BF16)
    ctx.softmax_backward(d_p, p, d_s, _rows(p), p.shape[-1], alpha=scale, stream=stream)
    d_q = matmul(ctx, d_s, k, stream=stream)
    d_k = matmul(ctx, d_s, q, True, False, stream=stream)
    return d_q, d_k, d_v


def split_heads(ctx, x, heads, *, stream=None) -> DeviceTensor:
    """[B, S, D] -> [B, H, S, dh] (reshape + transpose(1, 2), transformer_train.hpp:167-172)."""
    b, s, d = x.shape
    out = DeviceTensor(ctx, (b, heads, s, d // heads), BF16)
    ctx.permute(x, (b, s, heads, d // heads), (0, 2, 1, 3), out, stream=stream)
    return out


def merge_heads(ctx, x, *, stream=None) -> DeviceTensor:
    b, h, s, dh = x.shape
    out = DeviceTensor(ctx, (b, s, h * dh), BF16)
    ctx.permute(x, (b, h, s, dh), (0, 2, 1, 3), out, stream=stream)
    return out


def cross_entropy(ctx, logits, labels, *, need_grad=True, stream=None):
    """Mean cross-entropy over all rows; returns (loss scalar tensor fp32, d_logits or None)."""
    rows, classes = _rows(logits), logits.shape[-1]
    loss = DeviceTensor(ctx, (1,), F32)
    d_logits = DeviceTensor(ctx, logits.shape, BF16) if need_grad else None
    ctx.cross_entropy(logits, labels, rows, classes, loss_sum=loss, d_logits=d_logits, stream=stream)
    return loss, d_logits


def sgd_step(ctx, params, grads, lr, *, shadows=None, stream=None) -> None:
    """p <- p - lr * g. With fp32 master `params`, `shadows` are the bf16 copies the matmuls read."""
    ctx.sgd_step(params, grads, [p.numel for p in params], lr, p_dtype=params[0].dtype, g_dtype=grads[0].dtype,
                 shadows=shadows, stream=stream)


class Adam:
    """Adam with fp32 moments (py/optim.py:30-92 argument checks included)."""

    def __init__(self, ctx, params, *, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, shadows=None):
        if lr <= 0:
            raise ValueError("lr must be > 0")
        if eps <= 0:
            raise ValueError("eps must be > 0")
        if not isinstance(betas, (tuple, list)) or len(betas) != 2:
            raise ValueError("betas must be a tuple of (beta1, beta2)")
        if not (0.0 < betas[0] < 1.0 and 0.0 < betas[1] < 1.0):
            raise ValueError("betas must be in (0, 1)")
        self.ctx, self.params = ctx, list(params)
        self.shadows = list(shadows) if shadows else None
        self.lr, self.beta1, self.beta2, self.eps = float(lr), float(betas[0]), float(betas[1]), float(eps)
        self.m = [DeviceTensor.zeros(ctx, p.shape, F32) for p in self.params]
        self.v = [DeviceTensor.zeros(ctx, p.shape, F32) for p in self.params]
        # The step number lives on the device ({int64 step, two bias-correction factors}): a step that was recorded
        # into a trace then advances on every replay exactly like an eager step (py/optim.py:73-81 recurrence).
        self.state = DeviceTensor.zeros(ctx, (4,), F32)

    @property
    def t(self) -> int:
        """Steps taken so far (read back from the device)."""
        return int(self.state.numpy().view(np.int64)[0])

    def step(self, grads, *, indices=None, advance=True, stream=None) -> None:
        """One update. `indices` restricts it to those parameters (grads then lines up with indices): a step may be
        applied in several parts, e.g. while the gradients of the remaining parameters are still being averaged over
        the ranks; only the first part advances the step number (advance=False for the others)."""
        idx = list(range(len(self.params))) if indices is None else list(indices)
        pick = lambda items: [items[i] for i in idx]
        params = pick(self.params)
        self.ctx.adam_step_device(params, grads, pick(self.m), pick(self.v), [p.numel for p in params], self.state,
                                  advance=advance, lr=self.lr, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                                  p_dtype=params[0].dtype, g_dtype=grads[0].dtype,
                                  shadows=pick(self.shadows) if self.shadows else None, stream=stream)


# ---------------------------------------------------------------------------------------------------------------
# 2-layer MLP (TracedMLP<2>::train_step) with either MSE (the reference's loss) or cross-entropy
# ---------------------------------------------------------------------------------------------------------------
def mlp_train_step(ctx, x, target, params, lr, *, loss="ce", masters=None, stream=None):
    """Forward, loss, backward and SGD update of Linear -> ReLU -> Linear. `params` = [w1, b1, w2, b2] in bf16
    (what the matmuls read, updated in place); `masters`, when given, are their fp32 master copies: the update is
    applied to the masters and the bf16 tensors are refreshed from them in the same pass.
    Returns (loss before the update as an fp32 device scalar, gradients)."""
    w1, b1, w2, b2 = params
    h_pre = linear_forward(ctx, x, w1, b1, stream=stream)
    h = DeviceTensor(ctx, h_pre.shape, BF16)
    ctx.unary(capi.U_RELU, h_pre, h, h.numel, stream=stream)
    out = linear_forward(ctx, h, w2, b2, stream=stream)
    if loss == "ce":
        loss_t, d_out = cross_entropy(ctx, out, target, stream=stream)
    elif loss == "mse":
        # loss = mean((out - target)^2); d_out = 2 (out - target) / n
        diff = DeviceTensor(ctx, out.shape, BF16)
        ctx.binary(capi.B_SUB, out, out.shape, target, target.shape, diff, stream=stream)
        sq = DeviceTensor(ctx, out.shape, BF16)
        ctx.unary(capi.U_SQUARE, diff, sq, sq.numel, stream=stream)
        loss_bf = DeviceTensor(ctx, (1,), BF16)
        ctx.reduce(capi.R_MEAN, sq, 1, sq.numel, 1, loss_bf, stream=stream)
        loss_t = DeviceTensor(ctx, (1,), F32)
        ctx.cast(loss_bf, BF16, loss_t, F32, 1, stream=stream)
        d_out = DeviceTensor(ctx, out.shape, BF16)
        ctx.unary(capi.U_MUL_SCALAR, diff, d_out, d_out.numel, scalar=2.0 / out.numel, stream=stream)
    else:
        raise ValueError(loss)
    d_h, d_w2, d_b2 = linear_backward(ctx, h, w2, d_out, stream=stream)
    d_hpre = relu_backward(ctx, d_h, h_pre, stream=stream)
    _, d_w1, d_b1 = linear_backward(ctx, x, w1, d_hpre, need_dx=False, stream=stream)
    grads = [d_w1, d_b1, d_w2, d_b2]
    if masters is not None:
        sgd_step(ctx, masters, grads, lr, shadows=params, stream=stream)
    else:
        sgd_step(ctx, params, grads, lr, stream=stream)
    return loss_t, grads


# ---------------------------------------------------------------------------------------------------------------
# Pre-LN GPT-2 block (verify/compare_grads.py:37-97)
# ---------------------------------------------------------------------------------------------------------------
FUSED_HEAD_DIM = 64   # head dimension the fused attention kernels are built for


def _head_operands(ctx, t, heads, parts=1):
    """Per-head strided views of a [B, S, parts * H * dh] projection output: one b200_attn_operand per part, each
    addressing element (b, h, s, d) in place (no [B,S,H,dh] -> [B,H,S,dh] copy)."""
    b, s, width = t.shape
    dh = width // (parts * heads)
    return [ctx.attn_operand(t, s * width, dh, width, offset=i * heads * dh) for i in range(parts)]


def transformer_block_forward(ctx, x, w, heads, *, defer_add=False, stream=None):
    """x [B, S, D], or a pair (a, b) standing for a + b not yet summed (the sum then happens inside the first LayerNorm
    pass); w: dict with ln1_g, ln1_b, wq, bq, wk, bk, wv, bv, wo, bo, ln2_g, ln2_b, w1, b1, w2, b2, and
    optionally wqkv [3D, D] / bqkv [3D] (the three projections stacked, of which wq.. are then row views): one GEMM
    instead of three. With head dimension 64 the attention runs in the fused kernels on the projection outputs as
    they lie; other head dimensions take the materialised softmax path. Returns (out, cache); with defer_add the output
    is returned as the pair (residual, mlp_out) for the next consumer to sum."""
    if isinstance(x, tuple):
        x, ln1, mean1, rstd1 = add_layernorm_forward(ctx, x[0], x[1], w["ln1_g"], w["ln1_b"], stream=stream)
    else:
        ln1, mean1, rstd1 = layernorm_forward(ctx, x, w["ln1_g"], w["ln1_b"], stream=stream)
    b, s, d = x.shape
    dh = d // heads
    cache = dict(x=x, ln1=ln1, mean1=mean1, rstd1=rstd1)
    if dh == FUSED_HEAD_DIM:
        if "wqkv" in w:
            qkv = linear_forward(ctx, ln1, w["wqkv"], w["bqkv"], stream=stream)            # [B, S, 3D]
            q_op, k_op, v_op = _head_operands(ctx, qkv, heads, 3)
            cache["qkv"] = (qkv,)
        else:
            q, k, v = (linear_forward(ctx, ln1, w["w" + n], w["b" + n], stream=stream) for n in "qkv")
            (q_op,), (k_op,), (v_op,) = (_head_operands(ctx, t, heads) for t in (q, k, v))
            cache["qkv"] = (q, k, v)
        merged = DeviceTensor(ctx, (b, s, d), BF16)
        lse = DeviceTensor(ctx, (b, heads, s), F32)
        merged_lo = DeviceTensor(ctx, (b, s, d), BF16)      # what bf16 drops of the attention output: for the backward row term
        (o_op,), (olo_op,) = _head_operands(ctx, merged, heads), _head_operands(ctx, merged_lo, heads)
        ctx.attention_forward(q_op, k_op, v_op, o_op, lse, b, heads, s, head_dim=dh, causal=True, o_lo=olo_op, stream=stream)
        cache.update(lse=lse, merged_lo=merged_lo)
    else:
        q = split_heads(ctx, linear_forward(ctx, ln1, w["wq"], w["bq"], stream=stream), heads, stream=stream)
        k = split_heads(ctx, linear_forward(ctx, ln1, w["wk"], w["bk"], stream=stream), heads, stream=stream)
        v = split_heads(ctx, linear_forward(ctx, ln1, w["wv"], w["bv"], stream=stream), heads, stream=stream)
        attn, p = causal_attention_forward(ctx, q, k, v, stream=stream)
        merged = merge_heads(ctx, attn, stream=stream)
        cache.update(q=q, k=k, v=v, p=p)
    res1, ln2, mean2, rstd2 = add_layernorm_forward(ctx, x, linear_forward(ctx, merged, w["wo"], w["bo"], stream=stream),
                                                    w["ln2_g"], w["ln2_b"], stream=stream)
    h1 = linear_forward(ctx, ln2, w["w1"], w["b1"], stream=stream)
    h1g = DeviceTensor(ctx, h1.shape, BF16)
    ctx.unary(capi.U_GELU, h1, h1g, h1g.numel, stream=stream)
    mlp_out = linear_forward(ctx, h1g, w["w2"], w["b2"], stream=stream)
    cache.update(merged=merged, res1=res1, ln2=ln2, mean2=mean2, rstd2=rstd2, h1=h1, h1g=h1g)
    if defer_add:
        return (res1, mlp_out), cache
    return add(ctx, res1, mlp_out, stream=stream), cache


def transformer_block_backward(ctx, d_out, w, cache, heads, *, d_out_colsum=None, want_dx_colsum=False, stream=None):
    """Returns (dx, grads) with grads keyed like `w` (LayerNorm gradients are fp32, the rest bf16).
    d_out_colsum: column sums of d_out when the producer of d_out already has them (they are the FC2 bias gradient);
    want_dx_colsum: also return the column sums of dx as a third value, for the block below."""
    c, g = cache, {}
    b, s, d = c["x"].shape
    dh = d // heads
    d_h1g, g["w2"], g["b2"] = linear_backward(ctx, c["h1g"], w["w2"], d_out, need_db=d_out_colsum is None, stream=stream)
    if d_out_colsum is not None:
        g["b2"] = d_out_colsum
    d_h1, g["b1"] = gelu_backward(ctx, d_h1g, c["h1"], want_colsum=True, stream=stream)  # b1's gradient = column sums of d_h1
    d_ln2, g["w1"], _ = linear_backward(ctx, c["ln2"], w["w1"], d_h1, need_db=False, stream=stream)
    # d_res1 is the dY of the attention output projection: its column sums (from the same kernel) are that bias gradient
    d_res1, g["ln2_g"], g["ln2_b"], g["bo"] = layernorm_backward(ctx, d_ln2, c["res1"], w["ln2_g"], c["mean2"], c["rstd2"],
                                                                  upstream=d_out, want_colsum=True, stream=stream)
    d_merged, g["wo"], _ = linear_backward(ctx, c["merged"], w["wo"], d_res1, need_db=False, stream=stream)
    if "lse" in c:
        (o_op,), (do_op,) = _head_operands(ctx, c["merged"], heads), _head_operands(ctx, d_merged, heads)
        if len(c["qkv"]) == 1:
            q_op, k_op, v_op = _head_operands(ctx, c["qkv"][0], heads, 3)
            d_qkv = DeviceTensor(ctx, (b, s, 3 * d), BF16)
            dq_op, dk_op, dv_op = _head_operands(ctx, d_qkv, heads, 3)
            grads_in = (d_qkv,)
        else:
            (q_op,), (k_op,), (v_op,) = (_head_operands(ctx, t, heads) for t in c["qkv"])
            grads_in = tuple(DeviceTensor(ctx, (b, s, d), BF16) for _ in range(3))
            (dq_op,), (dk_op,), (dv_op,) = (_head_operands(ctx, t, heads) for t in grads_in)
        (olo_op,) = _head_operands(ctx, c["merged_lo"], heads)
        ctx.attention_backward(q_op, k_op, v_op, o_op, do_op, c["lse"], dq_op, dk_op, dv_op, b, heads, s, head_dim=dh,
                               causal=True, o_lo=olo_op, stream=stream)
    else:
        d_attn = split_heads(ctx, d_merged, heads, stream=stream)
        d_q, d_k, d_v = causal_attention_backward(ctx, c["q"], c["k"], c["v"], c["p"], d_attn, stream=stream)
        grads_in = tuple(merge_heads(ctx, t, stream=stream) for t in (d_q, d_k, d_v))
    if len(grads_in) == 1:
        d_ln1, g["wqkv"], g["bqkv"] = linear_backward(ctx, c["ln1"], w["wqkv"], grads_in[0], stream=stream)
        for i, n in enumerate("qkv"):
            g["w" + n], g["b" + n] = g["wqkv"].narrow0(i * d, d), g["bqkv"].narrow0(i * d, d)
    else:
        d_ln1_q, g["wq"], g["bq"] = linear_backward(ctx, c["ln1"], w["wq"], grads_in[0], stream=stream)
        d_ln1_k, g["wk"], g["bk"] = linear_backward(ctx, c["ln1"], w["wk"], grads_in[1], stream=stream)
        d_ln1_v, g["wv"], g["bv"] = linear_backward(ctx, c["ln1"], w["wv"], grads_in[2], stream=stream)
        d_ln1 = add(ctx, add(ctx, d_ln1_q, d_ln1_k, stream=stream), d_ln1_v, stream=stream)
    if want_dx_colsum:
        d_x, g["ln1_g"], g["ln1_b"], cs = layernorm_backward(ctx, d_ln1, c["x"], w["ln1_g"], c["mean1"], c["rstd1"],
                                                              upstream=d_res1, want_colsum=True, stream=stream)
        return d_x, g, cs
    d_x, g["ln1_g"], g["ln1_b"] = layernorm_backward(ctx, d_ln1, c["x"], w["ln1_g"], c["mean1"], c["rstd1"],
                                                      upstream=d_res1, stream=stream)
    return d_x, g


# ---------------------------------------------------------------------------------------------------------------
# GPT-2-shaped model: embeddings + L blocks + final LayerNorm + untied LM head + cross-entropy, Adam
# (TracedTransformerWithEmbedding, autograd/traced/transformer_train.hpp:363-507; bench/autograd/bench_gpt2_full.cpp)
# ---------------------------------------------------------------------------------------------------------------
BLOCK_KEYS = ("ln1_g", "ln1_b", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "ln2_g", "ln2_b", "w1", "b1", "w2", "b2")
_QKV_KEYS = ("wq", "bq", "wk", "bk", "wv", "bv")
_F32_GRADS = ("ln1_g", "ln1_b", "ln2_g", "ln2_b")   # LayerNorm gradients come out of their kernel in fp32


class GPT2:
    """Parameters live on the device in bf16; the vocabulary dimension is padded to a multiple of 8 rows so that
    logits rows start 16-byte aligned (50257 -> 50264); the cross-entropy kernel ignores the pad columns."""

    def __init__(self, ctx, *, layers, d_model, heads, seq, vocab, d_ff=None):
        self.ctx, self.L, self.D, self.H, self.S, self.V = ctx, layers, d_model, heads, seq, vocab
        self.F = d_ff or 4 * d_model
        self.Vp = (vocab + 7) // 8 * 8
        self.params = None
        self.opt = None
        self._d_logits = None

    def block_shapes(self):
        d, f = self.D, self.F
        return dict(ln1_g=(d,), ln1_b=(d,), wq=(d, d), bq=(d,), wk=(d, d), bk=(d,), wv=(d, d), bv=(d,), wo=(d, d), bo=(d,),
                    ln2_g=(d,), ln2_b=(d,), w1=(f, d), b1=(f,), w2=(d, f), b2=(d,))

    def load(self, host_params) -> None:
        """host_params: numpy arrays structured like the oracle's `gpt2_forward_backward` parameters."""
        import numpy as np
        ctx = self.ctx
        head = np.zeros((self.Vp, self.D), np.float32)
        head[: self.V] = host_params["head"]
        self.params = {
            "tok_emb": DeviceTensor.from_numpy(ctx, host_params["tok_emb"]),
            "pos_emb": DeviceTensor.from_numpy(ctx, host_params["pos_emb"]),
            "lnf_g": DeviceTensor.from_numpy(ctx, host_params["lnf_g"]),
            "lnf_b": DeviceTensor.from_numpy(ctx, host_params["lnf_b"]),
            "head": DeviceTensor.from_numpy(ctx, head),
            "blocks": [self._load_block(w) for w in host_params["blocks"]],
        }

    def _load_block(self, w):
        """The three attention projections are stored stacked ([3D, D] and [3D]) so that they run as one GEMM; wq, bq,
        ... stay addressable as row views of the stacked tensors."""
        import numpy as np
        ctx, d = self.ctx, self.D
        blk = {k: DeviceTensor.from_numpy(ctx, w[k]) for k in BLOCK_KEYS if k not in _QKV_KEYS}
        blk["wqkv"] = DeviceTensor.from_numpy(ctx, np.concatenate([w["wq"], w["wk"], w["wv"]], axis=0))
        blk["bqkv"] = DeviceTensor.from_numpy(ctx, np.concatenate([w["bq"], w["bk"], w["bv"]], axis=0))
        for i, n in enumerate("qkv"):
            blk["w" + n], blk["b" + n] = blk["wqkv"].narrow0(i * d, d), blk["bqkv"].narrow0(i * d, d)
        return blk

    def state(self) -> dict:
        """Host copy of the parameters in the structure `load` takes (fp32 numpy arrays holding the bf16 values; the
        padding rows of the LM head are dropped). load(state()) reproduces the device state bit for bit."""
        p = self.params
        out = {k: p[k].numpy() for k in ("tok_emb", "pos_emb", "lnf_g", "lnf_b")}
        out["head"] = p["head"].numpy()[: self.V]
        out["blocks"] = [{k: blk[k].numpy() for k in self.block_shapes()} for blk in p["blocks"]]
        return out

    def save(self, path) -> None:
        """Writes the parameters to one .npz file (keys `tok_emb`, ..., `blocks.<i>.<name>`): a weight dump for comparing
        two runs, or this implementation with another, tensor by tensor."""
        import numpy as np
        st = self.state()
        flat = {k: v for k, v in st.items() if k != "blocks"}
        for i, blk in enumerate(st["blocks"]):
            flat.update({f"blocks.{i}.{k}": v for k, v in blk.items()})
        np.savez(path, **flat)

    def load_file(self, path) -> None:
        """Loads a file written by `save`; the layer count and shapes must match this model."""
        import numpy as np
        with np.load(path) as z:
            names = set(z.files)
            blocks = [{k: z[f"blocks.{i}.{k}"] for k in self.block_shapes()} for i in range(self.L)]
            if f"blocks.{self.L}.w1" in names:
                raise ValueError(f"{path} holds more than {self.L} blocks")
            self.load({**{k: z[k] for k in ("tok_emb", "pos_emb", "lnf_g", "lnf_b", "head")}, "blocks": blocks})

    def init_random(self, seed=42, std=0.02) -> None:
        """N(0, std) weights, zero biases, LayerNorm gain 1 (random-init stand-in for a checkpoint)."""
        import numpy as np
        rng = np.random.default_rng(seed)

        def w(*shape):
            return (rng.standard_normal(shape, dtype=np.float32) * std)

        blocks = []
        for _ in range(self.L):
            blk = {}
            for k, shape in self.block_shapes().items():
                if k.endswith("_g"):
                    blk[k] = np.ones(shape, np.float32)
                elif len(shape) == 1:
                    blk[k] = np.zeros(shape, np.float32)
                else:
                    blk[k] = w(*shape)
            blocks.append(blk)
        self.load({"tok_emb": w(self.V, self.D), "pos_emb": w(self.S, self.D), "lnf_g": np.ones(self.D, np.float32),
                   "lnf_b": np.zeros(self.D, np.float32), "head": w(self.V, self.D), "blocks": blocks})

    def forward_backward(self, ids, targets, pos_ids, *, stream=None, segment_hook=None, blocks_per_segment=4):
        """ids, targets: uint32 device tensors [B, S] / [B*S]; pos_ids: uint32 [S] = 0..S-1.
        Returns (loss fp32 scalar tensor, grads structured like params).
        segment_hook(pairs), when given, is called with the (parameter, gradient) pairs that have just become final:
        after the LM head and final LayerNorm, after every `blocks_per_segment` blocks of the backward pass, and at the
        end with the remaining blocks (none when the count divides the depth) and the embeddings. A data-parallel driver ends a trace there and starts the
        all-reduce of those gradients while the rest of the backward pass runs."""
        ctx, p = self.ctx, self.params
        b = ids.numel // self.S
        t = b * self.S
        tok = DeviceTensor(ctx, (b, self.S, self.D), BF16)
        ctx.embedding_forward(ids, t, p["tok_emb"], self.V, self.D, tok, stream=stream)
        pos = DeviceTensor(ctx, (1, self.S, self.D), BF16)
        ctx.embedding_forward(pos_ids, self.S, p["pos_emb"], self.S, self.D, pos, stream=stream)
        x = add(ctx, tok, pos, stream=stream)
        caches = []
        for w in p["blocks"]:
            x, cache = transformer_block_forward(ctx, x, w, self.H, defer_add=True, stream=stream)
            caches.append(cache)
        if isinstance(x, tuple):   # the last block's residual sum happens inside the final LayerNorm pass
            x, xf, mean_f, rstd_f = add_layernorm_forward(ctx, x[0], x[1], p["lnf_g"], p["lnf_b"], stream=stream)
        else:
            xf, mean_f, rstd_f = layernorm_forward(ctx, x, p["lnf_g"], p["lnf_b"], stream=stream)
        logits = matmul(ctx, xf, p["head"], False, True, stream=stream)            # [B, S, Vp]
        loss = DeviceTensor(ctx, (1,), F32)
        # The cross-entropy kernel writes columns [0, V) only; the pad columns must be zero for the head gradient. The
        # buffer is kept across steps so that they are zeroed once, not every step.
        if self._d_logits is None or self._d_logits.shape != logits.shape:
            self._d_logits = DeviceTensor.zeros(ctx, logits.shape, BF16, stream=stream)
        d_logits = self._d_logits
        ctx.cross_entropy(logits, targets, t, self.V, ld=self.Vp, loss_sum=loss, d_logits=d_logits, ldd=self.Vp,
                          stream=stream)
        grads = {"blocks": [None] * self.L}
        d_xf, grads["head"], _ = linear_backward(ctx, xf, p["head"], d_logits, need_db=False, stream=stream)
        # every d_x below is the dY of the FC2 layer of the block it enters: its column sums travel with it
        d_x, grads["lnf_g"], grads["lnf_b"], d_x_cs = layernorm_backward(ctx, d_xf, x, p["lnf_g"], mean_f, rstd_f,
                                                                          want_colsum=True, stream=stream)
        if segment_hook:
            segment_hook([(p[k], grads[k]) for k in ("head", "lnf_g", "lnf_b")])
        pending, done = [], 0
        for i in reversed(range(self.L)):
            d_x, grads["blocks"][i], d_x_cs = transformer_block_backward(ctx, d_x, p["blocks"][i], caches[i], self.H,
                                                                         d_out_colsum=d_x_cs, want_dx_colsum=True, stream=stream)
            pending += [(p["blocks"][i][k], grads["blocks"][i][k]) for k in BLOCK_KEYS]
            done += 1
            if segment_hook and done % blocks_per_segment == 0:
                segment_hook(pending)
                pending = []
        grads["tok_emb"] = DeviceTensor(ctx, (self.V, self.D), F32)
        ctx.embedding_backward(ids, t, d_x, self.V, self.D, grads["tok_emb"], stream=stream)
        pos_g = DeviceTensor(ctx, (self.S, self.D), BF16)
        ctx.reduce(capi.R_SUM, d_x, 1, b, self.S * self.D, pos_g, stream=stream)
        grads["pos_emb"] = pos_g
        if segment_hook:
            segment_hook(pending + [(p["tok_emb"], grads["tok_emb"]), (p["pos_emb"], grads["pos_emb"])])
        return loss, grads

    def _flat(self, tree):
        """(bf16-gradient tensors, fp32-gradient tensors) in a fixed order, as (param, grad) pairs."""
        p = self.params
        bf, f32 = [], []
        f32.append((p["tok_emb"], tree["tok_emb"]))
        bf.append((p["pos_emb"], tree["pos_emb"]))
        f32.append((p["lnf_g"], tree["lnf_g"]))
        f32.append((p["lnf_b"], tree["lnf_b"]))
        bf.append((p["head"], tree["head"]))
        for w, g in zip(p["blocks"], tree["blocks"]):
            for k in BLOCK_KEYS:
                (f32 if k in _F32_GRADS else bf).append((w[k], g[k]))
        return bf, f32

    def adam_step(self, grads, *, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, stream=None) -> None:
        bf, f32 = self._flat(grads)
        if self.opt is None:
            self.opt = (Adam(self.ctx, [p for p, _ in bf], lr=lr, betas=betas, eps=eps),
                        Adam(self.ctx, [p for p, _ in f32], lr=lr, betas=betas, eps=eps))
        self.opt[0].step([g for _, g in bf], stream=stream)
        self.opt[1].step([g for _, g in f32], stream=stream)

    def num_params(self) -> int:
        bf, f32 = self._flat({"tok_emb": None, "pos_emb": None, "lnf_g": None, "lnf_b": None, "head": None,
                              "blocks": [dict.fromkeys(BLOCK_KEYS)] * self.L})
        return sum(p.numel for p, _ in bf + f32) - (self.Vp - self.V) * self.D
