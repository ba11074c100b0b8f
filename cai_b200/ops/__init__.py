"""Tensor-level wrappers over the sm_100a kernel library.

Each function takes CUDA ``torch.Tensor`` arguments, launches on the current stream and returns
its output tensor(s). There is no PyTorch fallback: these are the only implementation.
"""
from __future__ import annotations

import torch

from ._lib import KernelError, check, device_status, lib

EPI_BF16, EPI_F32, EPI_F32_ACCUM, EPI_BF16_RESIDUAL, EPI_SWIGLU, EPI_SWIGLU_BWD = 0, 1, 2, 3, 4, 5


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return t.data_ptr() if t is not None else None


def gemm(a, b, *, trans_a=False, trans_b=False, out=None, out_dtype=torch.bfloat16, accumulate=False,
         residual=None, alpha=1.0, sm_limit=0, seg_counts=None, seg_rows=0, seg_mode=0):
    """``C[M,N] = alpha * op(A) @ op(B)^T`` on the tcgen05 tensor cores.

    ``a`` is ``[M,K]`` (or ``[K,M]`` with ``trans_a``); ``b`` is ``[N,K]`` (or ``[K,N]`` with
    ``trans_b``). With ``out_dtype=torch.float32`` and ``accumulate`` the product is added to
    ``out``; ``residual`` (bf16 ``[M,N]``) is added in the epilogue.

    Ragged form (expert slabs): ``seg_counts`` (int32, one entry per ``seg_rows`` rows) gives the
    live rows of each sub-slab of M (``seg_mode=1``: tiles past the count are neither computed nor
    written) or of K (``seg_mode=2``: k-blocks past the count are skipped).
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    if trans_a:
        K, M = a.shape
    else:
        M, K = a.shape
    if trans_b:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"K mismatch {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), device=a.device, dtype=out_dtype)
    assert out.shape == (M, N) and out.stride(1) == 1
    if out.dtype == torch.bfloat16:
        epi = EPI_BF16_RESIDUAL if residual is not None else EPI_BF16
        assert not accumulate
    else:
        assert out.dtype == torch.float32 and residual is None
        epi = EPI_F32_ACCUM if accumulate else EPI_F32
    ldr = residual.stride(0) if residual is not None else 0
    if seg_counts is not None:
        assert seg_counts.dtype == torch.int32 and seg_mode in (1, 2) and seg_rows > 0
        check(lib().cai_gemm_bf16_seg(_p(a), _p(b), _p(out), _p(residual), M, N, K, a.stride(0), b.stride(0),
                                      out.stride(0), ldr, int(trans_a), int(trans_b), epi, float(alpha),
                                      _p(seg_counts), int(seg_rows), int(seg_mode), int(sm_limit), _stream()), "gemm_seg")
        return out
    check(lib().cai_gemm_bf16(_p(a), _p(b), _p(out), _p(residual), M, N, K, a.stride(0), b.stride(0),
                              out.stride(0), ldr, int(trans_a), int(trans_b), epi, float(alpha),
                              int(sm_limit), _stream()), "gemm")
    return out


def gemm_swiglu(x, wgu):
    """Gate/up projection with SwiGLU in the GEMM epilogue: ``gu = x @ wgu^T`` with ``wgu = [gate rows; up rows]``
    (``[2F, K]``, F a multiple of 128) and ``act = silu(gu[:, :F]) * gu[:, F:]``. Returns ``(gu, act)``."""
    assert x.dtype == torch.bfloat16 and wgu.dtype == torch.bfloat16 and x.stride(1) == 1 and wgu.stride(1) == 1
    M, K = x.shape
    N = wgu.shape[0]
    assert wgu.shape[1] == K and N % 256 == 0
    gu = torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
    act = torch.empty((M, N // 2), device=x.device, dtype=torch.bfloat16)
    check(lib().cai_gemm_bf16(_p(x), _p(wgu), _p(gu), _p(act), M, N, K, x.stride(0), wgu.stride(0), gu.stride(0), act.stride(0),
                              0, 0, EPI_SWIGLU, 1.0, 0, _stream()), "gemm_swiglu")
    return gu, act


def gemm_swiglu_bwd(dy, wd, gu):
    """Input gradient of the down projection with SwiGLU backward in the epilogue: ``dact = dy @ wd`` (``wd`` is
    ``[H, F]``) never reaches memory, the result is ``dgu = [dgate | dup]`` (``[T, 2F]``) from the saved ``gu``."""
    assert dy.dtype == torch.bfloat16 and wd.dtype == torch.bfloat16 and gu.dtype == torch.bfloat16
    M, K = dy.shape
    Kb, F = wd.shape
    assert K == Kb and gu.shape == (M, 2 * F) and gu.stride(1) == 1
    dgu = torch.empty((M, 2 * F), device=dy.device, dtype=torch.bfloat16)
    check(lib().cai_gemm_bf16(_p(dy), _p(wd), _p(dgu), _p(gu), M, F, K, dy.stride(0), wd.stride(0), dgu.stride(0), gu.stride(0),
                              0, 1, EPI_SWIGLU_BWD, 1.0, 0, _stream()), "gemm_swiglu_bwd")
    return dgu


def gemm_grouped(a, b, out, M, N, K, *, groups, trans_a=False, trans_b=False, accumulate=False, seg_counts=None, seg_rows=0,
                 seg_mode=0):
    """``groups`` products ``C_g[M,N] = op(A_g) @ op(B_g)^T`` in one launch; ``a``, ``b``, ``out`` hold the groups stacked
    along their row dimension (rows of ``[M,K]`` / ``[N,K]``, or of ``[K,M]`` / ``[K,N]`` when transposed)."""
    epi = (EPI_F32_ACCUM if accumulate else EPI_F32) if out.dtype == torch.float32 else EPI_BF16
    ga, gb = (K if trans_a else M), (K if trans_b else N)
    grp_seg = ((K if seg_mode == 2 else M) // seg_rows) if seg_mode else 0
    check(lib().cai_gemm_bf16_grouped(_p(a), _p(b), _p(out), M, N, K, a.stride(0), b.stride(0), out.stride(0), int(trans_a),
                                      int(trans_b), epi, _p(seg_counts), int(seg_rows), int(seg_mode), groups, ga, gb, M, grp_seg,
                                      _stream()), "gemm_grouped")
    return out


def moe_route_fwd(logits, k, cap):
    """Softmax top-k router. logits f32 ``[T,E]``. Returns ``idx`` int32 ``[T,k]``, ``w`` f32 ``[T,k]``
    (renormalised over the chosen k), ``pos`` int32 ``[T,k]`` (slot in the expert's slab, -1 when
    the expert already holds ``cap`` tokens) and ``counts`` int32 ``[E]``."""
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    idx = torch.empty(T, k, device=logits.device, dtype=torch.int32)
    pos = torch.empty_like(idx)
    w = torch.empty(T, k, device=logits.device, dtype=torch.float32)
    counts = torch.empty(E, device=logits.device, dtype=torch.int32)
    check(lib().cai_moe_route_fwd(_p(logits), _p(idx), _p(w), _p(pos), _p(counts), T, E, k, int(cap), _stream()), "moe_route_fwd")
    return idx, w, pos, counts


def moe_route_bwd(logits, idx, dw, pos):
    """Gradient of the router logits (bf16 ``[T,E]``) from the gradient of the combine weights."""
    T, E = logits.shape
    out = torch.empty(T, E, device=logits.device, dtype=torch.bfloat16)
    check(lib().cai_moe_route_bwd(_p(logits), _p(idx), _p(dw), _p(pos), _p(out), T, E, idx.shape[1], _stream()), "moe_route_bwd")
    return out


def rmsnorm_fwd(x, g, eps=1e-6):
    rows, H = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
    check(lib().cai_rmsnorm_fwd(_p(x), _p(g), _p(y), _p(rstd), rows, H, float(eps), _stream()), "rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(x, g, rstd, dy, dx=None, dg=None, dx_accumulate=False, dg_accumulate=False, scratch=None):
    rows, H = x.shape
    if dx is None:
        assert not dx_accumulate
        dx = torch.empty_like(x)
    if dg is None:
        assert not dg_accumulate
        dg = torch.empty(H, device=x.device, dtype=torch.float32)
    parts = lib().cai_rmsnorm_bwd_parts(rows)
    if scratch is None:
        scratch = torch.empty(parts * H, device=x.device, dtype=torch.float32)
    assert scratch.numel() >= parts * H
    check(lib().cai_rmsnorm_bwd(_p(x), _p(g), _p(rstd), _p(dy), _p(dx), _p(dg), _p(scratch), rows, H,
                                int(dx_accumulate), int(dg_accumulate), _stream()), "rmsnorm_bwd")
    return dx, dg


def rope_table(seq, hd, theta=10000.0, device="cuda"):
    t = torch.empty((seq, hd // 2, 2), device=device, dtype=torch.float32)
    check(lib().cai_rope_table(_p(t), seq, hd, float(theta), _stream()), "rope_table")
    return t


def rope_apply_(qkv, table, seq, nh, nkv, hd, inverse=False):
    T = qkv.shape[0]
    check(lib().cai_rope_apply(_p(qkv), _p(table), T, seq, nh, nkv, hd, qkv.stride(0), int(inverse), _stream()),
          "rope_apply")
    return qkv


def swiglu_fwd(gu):
    T, F2 = gu.shape
    act = torch.empty((T, F2 // 2), device=gu.device, dtype=gu.dtype)
    check(lib().cai_swiglu_fwd(_p(gu), _p(act), T, F2 // 2, _stream()), "swiglu_fwd")
    return act


def swiglu_bwd(gu, dact):
    T, F2 = gu.shape
    dgu = torch.empty_like(gu)
    check(lib().cai_swiglu_bwd(_p(gu), _p(dact), _p(dgu), T, F2 // 2, _stream()), "swiglu_bwd")
    return dgu


def embed_fwd(tokens, E, vocab_lo=0, vocab_hi=None):
    T = tokens.numel()
    H = E.shape[1]
    hi = vocab_lo + E.shape[0] if vocab_hi is None else vocab_hi
    out = torch.empty((T, H), device=E.device, dtype=E.dtype)
    check(lib().cai_embed_fwd(_p(tokens), _p(E), _p(out), T, H, vocab_lo, hi, _stream()), "embed_fwd")
    return out


def embed_bwd_(tokens, dout, dE, vocab_lo=0, vocab_hi=None):
    T = tokens.numel()
    H = dE.shape[1]
    hi = vocab_lo + dE.shape[0] if vocab_hi is None else vocab_hi
    check(lib().cai_embed_bwd(_p(tokens), _p(dout), _p(dE), T, H, vocab_lo, hi, _stream()), "embed_bwd")
    return dE


def cross_entropy_(logits, targets, loss_sum, grad_scale=1.0, loss_scale=1.0, row_lse=None):
    """In place: logits become dlogits; ``loss_sum`` (f32[1]) accumulates the scaled row losses."""
    rows, V = logits.shape
    check(lib().cai_cross_entropy(_p(logits), _p(targets), _p(loss_sum), _p(row_lse), rows, V, logits.stride(0),
                                  float(grad_scale), float(loss_scale), _stream()), "cross_entropy")
    return logits


def adamw_(master, m, v, grad, param, step, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.01, grad_scale=1.0):
    n = master.numel()
    check(lib().cai_adamw(_p(master), _p(m), _p(v), _p(grad), _p(param), n, float(lr), float(beta1), float(beta2),
                          float(eps), float(wd), float(grad_scale), int(step), _stream()), "adamw")


def flash_attn_fwd(qkv, B, S, nh, nkv, hd, scale=None, variant=0):
    """Causal GQA flash attention forward over packed ``qkv`` ``[B*S, (nh + 2 nkv) * hd]``. ``variant``: 0 = chosen
    from the grid size, 1 = one query tile per CTA (score MMA a block ahead), 2 = two tiles per CTA in ping-pong."""
    assert qkv.dtype == torch.bfloat16 and qkv.is_contiguous()
    scale = hd ** -0.5 if scale is None else scale
    out = torch.empty((B * S, nh * hd), device=qkv.device, dtype=torch.bfloat16)
    lse = torch.empty((B, nh, S), device=qkv.device, dtype=torch.float32)
    check(lib().cai_flash_attn_fwd_variant(_p(qkv), _p(out), _p(lse), B, S, nh, nkv, hd, float(scale), int(variant), _stream()),
          "flash_attn_fwd")
    return out, lse


def flash_attn_bwd(qkv, out, dout, lse, B, S, nh, nkv, hd, scale=None, dqkv=None, delta=None, parts=7):
    """Causal GQA flash attention backward. ``parts``: bit 0 delta, bit 1 dK / dV, bit 2 dQ."""
    scale = hd ** -0.5 if scale is None else scale
    if dqkv is None:
        dqkv = torch.empty_like(qkv)
    if delta is None:
        delta = torch.empty((B, nh, S), device=qkv.device, dtype=torch.float32)
    check(lib().cai_flash_attn_bwd_parts(_p(qkv), _p(out), _p(dout), _p(lse), _p(delta), _p(dqkv), B, S, nh, nkv, hd,
                                         float(scale), int(parts), _stream()), "flash_attn_bwd")
    return dqkv


__all__ = [n for n in dir() if not n.startswith("_")]


# ---------------------------------------------------------------------------- fp8 (e4m3) block-scaled GEMM
def quant_rows_1x128(x):
    """bf16 ``[rows, cols]`` -> (e4m3 ``[rows, cols]``, fp32 scales ``[rows, cols/128]``): one scale
    per row and 128 columns (``amax / 448``), the activation side of the block-scaled GEMM."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 128 == 0
    rows, cols = x.shape
    q = torch.empty(rows, cols, device=x.device, dtype=torch.float8_e4m3fn)
    s = torch.empty(rows, cols // 128, device=x.device, dtype=torch.float32)
    check(lib().cai_quant_rows_1x128(_p(x), x.stride(0), _p(q), cols, _p(s), rows, cols, _stream()), "quant_rows")
    return q, s


def quant_blocks_128x128(w, transposed=False):
    """bf16 ``[rows, cols]`` -> (e4m3 copy, fp32 scales ``[ceil(rows/128), ceil(cols/128)]``), one scale
    per 128x128 block (the weight side). With ``transposed`` also returns the e4m3 transpose
    ``[cols, rows]`` and its scale table, which the input-gradient GEMM consumes."""
    assert w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1
    rows, cols = w.shape
    nbr, nbc = (rows + 127) // 128, (cols + 127) // 128
    q = torch.empty(rows, cols, device=w.device, dtype=torch.float8_e4m3fn)
    s = torch.empty(nbr, nbc, device=w.device, dtype=torch.float32)
    qt = torch.empty(cols, rows, device=w.device, dtype=torch.float8_e4m3fn) if transposed else None
    st = torch.empty(nbc, nbr, device=w.device, dtype=torch.float32) if transposed else None
    check(lib().cai_quant_blocks_128x128(_p(w), w.stride(0), _p(q), cols, _p(qt), rows, _p(s), _p(st), rows, cols, _stream()),
          "quant_blocks")
    return (q, s, qt, st) if transposed else (q, s)


def gemm_fp8(aq, sa, bq, sb, *, out=None, out_dtype=torch.bfloat16, residual=None):
    """``C[M,N] = sum_kb sa[:,kb,None] * sb[n//128,kb] * (aq[:,kb] @ bq[:,kb]^T)`` on the tcgen05 tensor
    cores (kind::f8f6f4) with the per-block scale-and-add in the epilogue warps. ``aq`` ``[M,K]``,
    ``bq`` ``[N,K]`` e4m3; ``sa`` ``[M,K/128]``, ``sb`` ``[ceil(N/128),K/128]`` fp32."""
    M, K = aq.shape
    N, Kb = bq.shape
    assert K == Kb and K % 128 == 0 and aq.stride(1) == 1 and bq.stride(1) == 1
    assert sa.shape == (M, K // 128) and sb.shape == ((N + 127) // 128, K // 128) and sa.is_contiguous() and sb.is_contiguous()
    if out is None:
        out = torch.empty(M, N, device=aq.device, dtype=out_dtype)
    epi = EPI_F32 if out.dtype == torch.float32 else (EPI_BF16_RESIDUAL if residual is not None else EPI_BF16)
    check(lib().cai_gemm_fp8_blockscaled(_p(aq), _p(sa), _p(bq), _p(sb), _p(out), _p(residual), M, N, K, aq.stride(0), bq.stride(0),
                                         out.stride(0), residual.stride(0) if residual is not None else 0, epi, _stream()), "gemm_fp8")
    return out
