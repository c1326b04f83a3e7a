"""Torch-tensor front end of the C ABI: each function borrows device pointers from its
arguments, launches on torch's current stream and returns torch tensors.  Nothing here
computes on the host and nothing falls back to PyTorch arithmetic."""

from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import numpy as np
import torch

from . import _lib

BF16 = torch.bfloat16


class KernelTimer:
    """Optional CUDA-event timing of one kernel family on the launching stream.  Set
    `ops.GEMM_TIMER = KernelTimer()` to collect; reading the total synchronises."""

    def __init__(self):
        self.events, self.flops, self.launches = [], 0, 0

    def start(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def stop(self, begin, flops):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.events.append((begin, e))
        self.flops += flops
        self.launches += 1

    def total_ms(self):
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self.events)


GEMM_TIMER = None
ATTN_TIMER = None


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _need(t, name, dtype=BF16):
    if not t.is_cuda:
        raise ValueError(f'{name} must live on a CUDA device (there is no CPU path)')
    if t.dtype != dtype:
        raise ValueError(f'{name} must be {dtype}, got {t.dtype}')
    return t


def _rows(t, name, dtype=BF16):
    """View [..., h] as rows with one stride; returns (tensor, rows, h, row_stride)."""
    _need(t, name, dtype)
    if t.stride(-1) != 1:
        raise ValueError(f'{name} must be contiguous in its last dimension')
    flat = t.reshape(-1, t.shape[-1])
    return flat, flat.shape[0], flat.shape[1], (flat.stride(0) if flat.shape[0] > 1 else flat.shape[1])


def device_check():
    lib = _lib.load()
    _lib.check(lib.bg_device_check(), 'bg_device_check')


def read_status():
    """Synchronise the current stream and raise if a bounded device wait ran out."""
    lib = _lib.load()
    code = lib.bg_read_status(_stream())
    if code != 0:
        raise _lib.B200Error(f'device status {code}: {lib.bg_last_error_string().decode()}')


def rmsnorm(x, weight, eps=1e-6):
    """rmsnorm(x) * (1 + weight) as bf16; x bf16, or fp32 (the fp32 residual stream; hidden size a multiple of 256)."""
    lib = _lib.load()
    fp32 = x.dtype == torch.float32
    flat, rows, h, ldx = _rows(x, 'x', x.dtype if fp32 else BF16)
    if fp32 and h % 256:
        raise ValueError('an fp32 input needs a hidden size that is a multiple of 256')
    out = torch.empty((rows, h), device=x.device, dtype=BF16)
    entry, name = (lib.bg_rmsnorm_f32, 'bg_rmsnorm_f32') if fp32 else (lib.bg_rmsnorm, 'bg_rmsnorm')
    _lib.check(entry(_ptr(flat), ldx, _ptr(_need(weight, 'weight')), _ptr(out), h, rows, h, eps, _stream()), name)
    return out.view(x.shape)


def add_rmsnorm_(y, w_post, resid, w_next=None, eps=1e-6):
    """resid += rmsnorm(y)*(1+w_post) in place; returns rmsnorm(resid)*(1+w_next) (bf16) or None.
    resid is bf16 (post-norm result and sum each rounded to bf16, as the module chain does) or fp32
    (nothing rounded on the way into the residual stream)."""
    lib = _lib.load()
    fp32 = resid.dtype == torch.float32
    fp32_y = y.dtype == torch.float32
    if fp32_y and not fp32:
        raise ValueError('an fp32 y needs an fp32 residual stream')
    _need(y, 'y', y.dtype if fp32_y else BF16), _need(resid, 'resid', resid.dtype if fp32 else BF16)
    if not (y.is_contiguous() and resid.is_contiguous()) or y.shape != resid.shape:
        raise ValueError('y and resid must be contiguous and of equal shape')
    h = y.shape[-1]
    if fp32 and h % 256:
        raise ValueError('an fp32 residual stream needs a hidden size that is a multiple of 256')
    rows = y.numel() // h
    normed = torch.empty(y.shape, device=y.device, dtype=BF16) if w_next is not None else None
    entry, name = ((lib.bg_add_rmsnorm_f32y, 'bg_add_rmsnorm_f32y') if fp32_y else
                   (lib.bg_add_rmsnorm_f32, 'bg_add_rmsnorm_f32') if fp32 else (lib.bg_add_rmsnorm, 'bg_add_rmsnorm'))
    _lib.check(entry(_ptr(y), _ptr(_need(w_post, 'w_post')), _ptr(resid), _ptr(w_next), _ptr(normed),
                     rows, h, eps, _stream()), name)
    return normed


@lru_cache(maxsize=32)
def inv_freq(head_dim, theta, device):
    """theta^(-2i/D) in fp32, computed the way the rotary module does
    (transformers modeling_t5gemma2.py:147-150)."""
    value = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    return value.to(device)


def qk_norm_rope_(q, k, q_weight, k_weight, positions, freqs, eps=1e-6, rotate=True, table=None):
    """In place on q [T,Hq,D] and k [T,Hkv,D] (views with a token stride are fine).  `table` (from
    rope_table, covering every position in use) replaces the per-token sincosf by a lookup of the same
    values; `freqs` is then not read."""
    lib = _lib.load()
    if rotate and table is not None:
        tokens, head_dim = q.shape[0], q.shape[-1]
        for t, name in ((q, 'q'), (k, 'k')):
            _need(t, name)
            if t.stride(-1) != 1 or t.stride(1) != head_dim:
                raise ValueError(f'{name} heads must be contiguous [T, heads, D]')
        _need(positions, 'positions', torch.int32), _need(table, 'rope table', torch.float32)
        if table.shape[1:] != (head_dim // 2, 2) or not table.is_contiguous() or positions.numel() != tokens:
            raise ValueError('the table must be [rows, head_dim/2, 2] and positions must have one entry per token')
        _lib.check(lib.bg_qk_norm_rope_cached(_ptr(q), q.stride(0), q.shape[1], _ptr(k), k.stride(0), k.shape[1],
                                              _ptr(_need(q_weight, 'q_weight')), _ptr(_need(k_weight, 'k_weight')),
                                              _ptr(positions), _ptr(table), table.shape[0], tokens, head_dim, eps,
                                              _stream()), 'bg_qk_norm_rope_cached')
        return
    ref = q if q is not None else k
    tokens, head_dim = ref.shape[0], ref.shape[-1]
    for t, name in ((q, 'q'), (k, 'k')):
        if t is not None:
            _need(t, name)
            if t.stride(-1) != 1 or t.stride(1) != head_dim:
                raise ValueError(f'{name} heads must be contiguous [T, heads, D]')
    if rotate:
        _need(positions, 'positions', torch.int32), _need(freqs, 'inv_freq', torch.float32)
    _lib.check(lib.bg_qk_norm_rope(
        _ptr(q), q.stride(0) if q is not None else 0, q.shape[1] if q is not None else 0,
        _ptr(k), k.stride(0) if k is not None else 0, k.shape[1] if k is not None else 0,
        _ptr(q_weight), _ptr(k_weight), _ptr(positions) if rotate else 0, _ptr(freqs) if rotate else 0,
        tokens, head_dim, eps, 1 if rotate else 0, _stream()), 'bg_qk_norm_rope')


def qk_norm_rope_table_(q, k, q_weight, k_weight, cos, sin, eps=1e-6):
    """In place on q [T,Hq,D], k [T,Hkv,D] with bf16 cos / sin tables [T, D]."""
    lib = _lib.load()
    tokens, head_dim = q.shape[0], q.shape[-1]
    for t, name in ((q, 'q'), (k, 'k')):
        _need(t, name)
        if t.stride(-1) != 1 or t.stride(1) != head_dim:
            raise ValueError(f'{name} heads must be contiguous [T, heads, D]')
    cos, sin = _need(cos, 'cos').contiguous(), _need(sin, 'sin').contiguous()
    if cos.shape != (tokens, head_dim) or sin.shape != (tokens, head_dim):
        raise ValueError(f'cos/sin must be [{tokens}, {head_dim}]')
    _lib.check(lib.bg_qk_norm_rope_table(_ptr(q), q.stride(0), q.shape[1], _ptr(k), k.stride(0), k.shape[1],
                                         _ptr(_need(q_weight, 'q_weight')), _ptr(_need(k_weight, 'k_weight')),
                                         _ptr(cos), _ptr(sin), tokens, head_dim, eps, _stream()),
               'bg_qk_norm_rope_table')


def embed(ids, table, eoi_embedding, scale, eoi_token=256_000, dtype=BF16):
    """table[ids] * scale (the end-of-image row unscaled); dtype torch.float32 writes an fp32 residual stream."""
    lib = _lib.load()
    _need(ids, 'ids', torch.int64), _need(table, 'table')
    if dtype not in (BF16, torch.float32):
        raise ValueError('the embedding is written as bf16 or fp32')
    ids = ids.reshape(-1).contiguous()
    out = torch.empty((ids.numel(), table.shape[1]), device=table.device, dtype=dtype)
    entry, name = (lib.bg_embed, 'bg_embed') if dtype == BF16 else (lib.bg_embed_f32, 'bg_embed_f32')
    _lib.check(entry(_ptr(ids), _ptr(table), _ptr(_need(eoi_embedding, 'eoi_embedding')), _ptr(out),
                     ids.numel(), table.shape[1], scale, eoi_token, table.shape[0], _stream()), name)
    return out


SPLIT_K = True      # latency path: allow K slices for under-filled problems (microbench turns it off to compare)


def _gemm(lib, few_rows, m, n, k, epilogue):
    """The entry point for a contraction: the weight-streaming kernel when the caller allows it
    (`few_rows`) and the shape is one it takes, else the throughput kernels."""
    if few_rows and lib.bg_gemm_bf16_skinny_supported(m, n, k, epilogue):
        return lib.bg_gemm_bf16_skinny, 'bg_gemm_bf16_skinny'
    return lib.bg_gemm_bf16, 'bg_gemm_bf16'


def linear(x, weight, out=None, *, few_rows=False):
    """x [..., K] @ weight[N, K].T -> [..., N] on the tensor cores.  `few_rows=True` is the latency path:
    inputs of up to 256 rows take the weight-streaming cluster split-K kernel, a few hundred rows against a
    narrow weight with a long contraction take the CTA-pair kernel with K slices as extra work items
    (fp32 summation order differs from the throughput kernels in both)."""
    lib = _lib.load()
    flat, m, k, lda = _rows(x, 'x')
    _need(weight, 'weight')
    if weight.ndim != 2 or weight.shape[1] != k or weight.stride(1) != 1:
        raise ValueError(f'weight must be [N, {k}] with contiguous rows')
    n = weight.shape[0]
    if out is None:
        out = torch.empty((m, n), device=x.device, dtype=BF16)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    split = lib.bg_gemm_bf16_splitk_choice(m, n, k) if few_rows and SPLIT_K and m > 256 else 1
    if split > 1:
        # a few hundred rows against a narrow weight: K slices as extra work items, fp32 partials summed once
        need = lib.bg_gemm_bf16_splitk_workspace_bytes(m, n, split)
        work = torch.empty((need,), device=x.device, dtype=torch.uint8)
        _lib.check(lib.bg_gemm_bf16_splitk(_ptr(flat), lda, _ptr(weight), weight.stride(0), _ptr(out), out.stride(0),
                                           m, n, k, split, _ptr(work), need, _stream()), 'bg_gemm_bf16_splitk')
    else:
        fn, name = _gemm(lib, few_rows, m, n, k, 0)
        _lib.check(fn(_ptr(flat), lda, _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), m, n, k, 0, _stream()), name)
    if timer is not None:
        timer.stop(begin, 2 * m * n * k)
    return out.view(*x.shape[:-1], n)


_ROPE_TABLES = {}


def linear_f32out(x, weight):
    """F.linear(x, weight) with the fp32 accumulators returned unrounded (fp32 [..., N])."""
    lib = _lib.load()
    flat, m, k, ldx = _rows(x, 'x')
    _need(weight, 'weight')
    n = weight.shape[0]
    if weight.shape[1] != k or weight.stride(1) != 1:
        raise ValueError('weight must be [N, K] with a contiguous last dimension')
    out = torch.empty((m, n), device=x.device, dtype=torch.float32)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    _lib.check(lib.bg_gemm_bf16_f32out(_ptr(flat), ldx, _ptr(weight), weight.stride(0), _ptr(out), m, n, k, _stream()),
               'bg_gemm_bf16_f32out')
    if timer is not None:
        timer.stop(begin, 2 * m * n * k)
    return out.view(*x.shape[:-1], n)


def rope_table(head_dim, theta, rows, device):
    """(cos, sin) fp32 [rows', head_dim/2, 2] of position * inv_freq for positions below rows' >= rows
    (grown in powers of two, one table per (head_dim, theta, device))."""
    key = (int(head_dim), float(theta), str(device))
    table = _ROPE_TABLES.get(key)
    if table is None or table.shape[0] < rows:
        size = 8192
        while size < rows:
            size *= 2
        table = torch.empty((size, head_dim // 2, 2), device=device, dtype=torch.float32)
        _lib.check(_lib.load().bg_rope_table(_ptr(table), size, head_dim, _ptr(inv_freq(head_dim, theta, device)),
                                             _stream()), 'bg_rope_table')
        _ROPE_TABLES[key] = table
    return table


def linear_qkv_rope(x, weight, q_dim, kv_dim, head_dim, q_weight, k_weight, positions, table, eps=1e-6):
    """x [T, K] @ [Wq; Wk; Wv].T -> [T, q_dim + 2 kv_dim] with QK-norm + RoPE applied to the query and
    key heads inside the GEMM epilogue (value heads untouched)."""
    lib = _lib.load()
    flat, m, k, lda = _rows(x, 'x')
    _need(weight, 'weight'), _need(positions, 'positions', torch.int32), _need(table, 'rope table', torch.float32)
    n = q_dim + 2 * kv_dim
    if weight.shape != (n, k) or weight.stride(1) != 1:
        raise ValueError(f'weight must be [{n}, {k}] with contiguous rows')
    if positions.numel() != m or table.shape[1:] != (head_dim // 2, 2) or not table.is_contiguous():
        raise ValueError('positions must have one entry per row and the table must be [rows, head_dim/2, 2]')
    out = torch.empty((m, n), device=x.device, dtype=BF16)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    _lib.check(lib.bg_gemm_bf16_qkv_rope(_ptr(flat), lda, _ptr(weight), weight.stride(0), _ptr(out), n, m, k, q_dim,
                                         kv_dim, head_dim, _ptr(_need(q_weight, 'q_norm')), _ptr(_need(k_weight, 'k_norm')),
                                         _ptr(positions), _ptr(table), table.shape[0], eps, _stream()),
               'bg_gemm_bf16_qkv_rope')
    if timer is not None:
        timer.stop(begin, 2 * m * n * k)
    return out


def linear_geglu(x, gate_up, *, few_rows=False):
    """gelu_tanh(x @ gate.T) * (x @ up.T) with gate_up = cat([gate, up]) of shape [2I, K]."""
    lib = _lib.load()
    flat, m, k, lda = _rows(x, 'x')
    _need(gate_up, 'gate_up')
    if gate_up.ndim != 2 or gate_up.shape[1] != k or gate_up.shape[0] % 2 or gate_up.stride(1) != 1:
        raise ValueError(f'gate_up must be [2I, {k}] with contiguous rows')
    n = gate_up.shape[0] // 2
    out = torch.empty((m, n), device=x.device, dtype=BF16)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    fn, name = _gemm(lib, few_rows, m, n, k, 1)
    _lib.check(fn(_ptr(flat), lda, _ptr(gate_up), gate_up.stride(0), _ptr(out), n, m, n, k, 1, _stream()), name)
    if timer is not None:
        timer.stop(begin, 4 * m * n * k)
    return out.view(*x.shape[:-1], n)


def transpose(x, pad_to=8):
    """x [R, C] -> contiguous [C, R'] with R' = R rounded up to `pad_to` (zero padded): the layout the
    GEMM needs when the contraction runs over R."""
    lib = _lib.load()
    _need(x, 'x')
    if x.ndim != 2 or x.stride(1) != 1:
        raise ValueError('transpose takes a 2-D tensor with contiguous rows')
    r, c = x.shape
    rp = (r + pad_to - 1) // pad_to * pad_to
    out = (torch.zeros if rp != r else torch.empty)((c, rp), device=x.device, dtype=BF16)
    _lib.check(lib.bg_transpose_bf16(_ptr(x), x.stride(0), _ptr(out), rp, r, c, _stream()), 'bg_transpose_bf16')
    return out


def linear_backward(x, weight, dy, *, need_dx=True, need_dw=True):
    """Gradients of y = x @ weight.T: dx = dy @ weight, dw = dy.T @ x, both on the tensor cores."""
    flat, m, k, _ = _rows(x, 'x')
    n = weight.shape[0]
    dy2 = dy.reshape(m, n)
    if dy2.stride(1) != 1:
        dy2 = dy2.contiguous()
    dx = dw = None
    if need_dx:
        dx = linear(dy2, transpose(weight)).view(x.shape)             # contraction over N
    if need_dw:
        dw = linear_tn(dy2, flat)                                     # contraction over the rows, operands as they lie
    return dx, dw


def linear_tn(at, wt):
    """at [R, M], wt [R, N] -> at.T @ wt [M, N]: the contraction runs over the rows of both operands, which the
    tensor core reads as MN-major tiles (no transposed copies).  Shapes the entry point does not take (M or N
    not a multiple of 8, misaligned views) go through explicit transposes."""
    lib = _lib.load()
    _need(at, 'at'), _need(wt, 'wt')
    if at.ndim != 2 or wt.ndim != 2 or at.shape[0] != wt.shape[0] or at.stride(1) != 1 or wt.stride(1) != 1:
        raise ValueError('linear_tn takes two 2-D tensors with contiguous rows and the same number of rows')
    r, m = at.shape
    n = wt.shape[1]
    direct = (m % 8 == 0 and n % 8 == 0 and at.stride(0) % 8 == 0 and wt.stride(0) % 8 == 0
              and at.data_ptr() % 16 == 0 and wt.data_ptr() % 16 == 0 and r > 0)
    if not direct:
        return linear(transpose(at), transpose(wt))
    out = torch.empty((m, n), device=at.device, dtype=BF16)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    split = lib.bg_gemm_bf16_splitk_choice(m, n, r) if SPLIT_K else 1
    need = lib.bg_gemm_bf16_splitk_workspace_bytes(m, n, split)
    work = torch.empty((need,), device=at.device, dtype=torch.uint8) if need else None
    _lib.check(lib.bg_gemm_bf16_tn(_ptr(at), at.stride(0), _ptr(wt), wt.stride(0), _ptr(out), n, m, n, r, split,
                                   _ptr(work), need, _stream()), 'bg_gemm_bf16_tn')
    if timer is not None:
        timer.stop(begin, 2 * m * n * r)
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return linear(x, weight)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dx, dw = linear_backward(x, weight, dy, need_dx=ctx.needs_input_grad[0], need_dw=ctx.needs_input_grad[1])
        return dx, dw


GEGLU_KEEP_PREACTIVATIONS = True


class _LinearGeglu(torch.autograd.Function):
    """h = gelu_tanh(x Wg^T) * (x Wu^T).  With GEGLU_KEEP_PREACTIVATIONS (default) the forward writes the bf16
    pre-activations [g | u] with the plain GEMM, forms h in a second pass and keeps [g | u] for the backward,
    as the native module does; without it the fused GEMM + GeGLU epilogue runs and the backward recomputes
    [g | u] with one more GEMM (they are four times the size of x)."""

    @staticmethod
    def forward(ctx, x, gate_up):
        if not GEGLU_KEEP_PREACTIVATIONS:
            ctx.save_for_backward(x, gate_up)
            ctx.kept = False
            return linear_geglu(x, gate_up)
        lib = _lib.load()
        flat, m, k, _ = _rows(x, 'x')
        inter = gate_up.shape[0] // 2
        gu = linear(flat, gate_up)
        h = torch.empty((m, inter), device=x.device, dtype=BF16)
        _lib.check(lib.bg_geglu_forward(_ptr(gu), _ptr(h), m, inter, _stream()), 'bg_geglu_forward')
        ctx.save_for_backward(x, gate_up, gu)
        ctx.kept = True
        return h.view(*x.shape[:-1], inter)

    @staticmethod
    def backward(ctx, dh):
        lib = _lib.load()
        if ctx.kept:
            x, gate_up, gu = ctx.saved_tensors
            flat, m, k, _ = _rows(x, 'x')
        else:
            x, gate_up = ctx.saved_tensors
            flat, m, k, _ = _rows(x, 'x')
            gu = linear(flat, gate_up)
        inter = gate_up.shape[0] // 2
        dh2 = dh.reshape(m, inter).contiguous()
        dgu = torch.empty_like(gu)
        _lib.check(lib.bg_geglu_backward(_ptr(gu), _ptr(dh2), _ptr(dgu), m, inter, _stream()), 'bg_geglu_backward')
        dx, dw = linear_backward(x, gate_up, dgu, need_dx=ctx.needs_input_grad[0], need_dw=ctx.needs_input_grad[1])
        return dx, dw


def rmsnorm_backward(x, weight, dy, eps=1e-6):
    """(dx bf16 like x, dw fp32 [h]) of y = rmsnorm(x) * (1 + weight)."""
    lib = _lib.load()
    flat, rows, h, ldx = _rows(x, 'x')
    dflat, drows, dh, lddy = _rows(dy.to(BF16), 'dy')
    if (drows, dh) != (rows, h):
        raise ValueError('dy must have the shape of x')
    dx = torch.empty((rows, h), device=x.device, dtype=BF16)
    dw = torch.empty((h,), device=x.device, dtype=torch.float32)
    need = lib.bg_rmsnorm_backward_workspace_bytes(rows, h)
    work = torch.empty((max(need, 4),), device=x.device, dtype=torch.uint8)
    _lib.check(lib.bg_rmsnorm_backward(_ptr(flat), ldx, _ptr(_need(weight, 'weight')), _ptr(dflat), lddy, _ptr(dx), h,
                                       _ptr(dw), _ptr(work), need, rows, h, eps, _stream()), 'bg_rmsnorm_backward')
    return dx.view(x.shape), dw


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        w = weight.detach().to(BF16)
        ctx.save_for_backward(x, w)
        ctx.eps, ctx.weight_dtype = eps, weight.dtype
        return rmsnorm(x, w, eps)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx, dw = rmsnorm_backward(x, w, dy.contiguous(), ctx.eps)
        return dx, dw.to(ctx.weight_dtype), None


def rmsnorm_autograd(x, weight, eps=1e-6):
    """rmsnorm() that records its backward (input and gain gradients from one kernel pass)."""
    return _RmsNorm.apply(x if x.stride(-1) == 1 else x.contiguous(), weight, eps)


def qk_norm_rope_backward(xq, xk, q_weight, k_weight, dyq, dyk, *, positions=None, freqs=None, cos=None, sin=None,
                          eps=1e-6, rotate=True, out_q=None, out_k=None):
    """Backward of qk_norm_rope_ / qk_norm_rope_table_: xq [T,Hq,D] and xk [T,Hkv,D] (or None) are the inputs
    the forward normalised, dyq / dyk the gradients of its outputs.  Returns (dxq, dxk, dq_weight, dk_weight)
    with fp32 gain gradients; the k entries are None when xk is None.  out_q / out_k ([T, heads, D] views with
    contiguous heads, e.g. slices of one gradient buffer of the stacked projection) receive dxq / dxk in place."""
    lib = _lib.load()
    tokens, hq, d = xq.shape

    def token_major(t, name):
        _need(t, name)
        if t.stride(-1) != 1 or t.stride(1) != d:
            t = t.contiguous()
        return t

    xq, dyq = token_major(xq, 'xq'), token_major(dyq.to(BF16), 'dyq')
    dxq = out_q if out_q is not None else torch.empty((tokens, hq, d), device=xq.device, dtype=BF16)
    dqw = torch.empty((d,), device=xq.device, dtype=torch.float32)
    hk = 0
    dxk = dkw = None
    if xk is not None:
        hk = xk.shape[1]
        xk, dyk = token_major(xk, 'xk'), token_major(dyk.to(BF16), 'dyk')
        dxk = out_k if out_k is not None else torch.empty((tokens, hk, d), device=xq.device, dtype=BF16)
        dkw = torch.empty((d,), device=xq.device, dtype=torch.float32)
    if rotate and cos is None:
        _need(positions, 'positions', torch.int32), _need(freqs, 'inv_freq', torch.float32)
    if cos is not None:
        cos, sin = _need(cos, 'cos').contiguous(), _need(sin, 'sin').contiguous()
        if cos.shape != (tokens, d) or sin.shape != (tokens, d):
            raise ValueError(f'cos/sin must be [{tokens}, {d}]')
    need = lib.bg_qk_norm_rope_backward_workspace_bytes(tokens, d)
    work = torch.empty((max(need, 4),), device=xq.device, dtype=torch.uint8)
    stride = lambda t: t.stride(0) if t is not None else 0
    _lib.check(lib.bg_qk_norm_rope_backward(
        _ptr(xq), stride(xq), _ptr(dyq), stride(dyq), _ptr(dxq), stride(dxq), hq,
        _ptr(xk), stride(xk), _ptr(dyk) if xk is not None else 0, stride(dyk) if xk is not None else 0, _ptr(dxk),
        stride(dxk), hk, _ptr(_need(q_weight, 'q_weight')), _ptr(k_weight), _ptr(positions) if positions is not None else 0,
        _ptr(freqs) if freqs is not None else 0, _ptr(cos), _ptr(sin), _ptr(dqw), _ptr(dkw), _ptr(work), need, tokens, d,
        eps, 1 if rotate else 0, _stream()), 'bg_qk_norm_rope_backward')
    return dxq, dxk, dqw, dkw


class _QkNormRope(torch.autograd.Function):
    """Out-of-place QK-norm + RoPE with its backward; angles from bf16 cos / sin tables [T, D] or from
    positions (int32 [T]) and inverse frequencies."""

    @staticmethod
    def forward(ctx, q, k, q_weight, k_weight, cos, sin, positions, freqs, eps):
        qw, kw = q_weight.detach().to(BF16), k_weight.detach().to(BF16)
        ctx.save_for_backward(q, k, qw, kw)
        # angle sources carry no gradient and may be cached tensors made under inference mode: kept as attributes
        ctx.angles = (cos, sin, positions, freqs)
        ctx.eps, ctx.dtypes = eps, (q_weight.dtype, k_weight.dtype)
        q2, k2 = q.clone(memory_format=torch.contiguous_format), k.clone(memory_format=torch.contiguous_format)
        if cos is not None:
            qk_norm_rope_table_(q2, k2, qw, kw, cos, sin, eps)
        else:
            qk_norm_rope_(q2, k2, qw, kw, positions, freqs, eps)
        return q2, k2

    @staticmethod
    def backward(ctx, dq, dk):
        q, k, qw, kw = ctx.saved_tensors
        cos, sin, positions, freqs = ctx.angles
        dxq, dxk, dqw, dkw = qk_norm_rope_backward(q, k, qw, kw, dq, dk, positions=positions, freqs=freqs, cos=cos,
                                                   sin=sin, eps=ctx.eps)
        return dxq, dxk, dqw.to(ctx.dtypes[0]), dkw.to(ctx.dtypes[1]), None, None, None, None, None


class _QkvNormRope(torch.autograd.Function):
    """The stacked projection output qkv [T, (Hq + 2 Hkv) D] -> (q', k', v) with QK-norm + RoPE on q and k.  One
    function instead of three slices plus _QkNormRope so that the backward writes the three gradients into ONE
    buffer shaped like qkv (the kernel takes row strides), not into zero-filled copies that autograd then adds."""

    @staticmethod
    def forward(ctx, qkv, q_heads, kv_heads, d, q_weight, k_weight, cos, sin, positions, freqs, eps):
        qw, kw = q_weight.detach().to(BF16), k_weight.detach().to(BF16)
        t, qd, kd = qkv.shape[0], q_heads * d, kv_heads * d
        ctx.save_for_backward(qkv, qw, kw)
        ctx.angles = (cos, sin, positions, freqs)
        ctx.meta = (q_heads, kv_heads, d, eps, q_weight.dtype, k_weight.dtype)
        q = qkv[:, :qd].reshape(t, q_heads, d).contiguous()
        k = qkv[:, qd:qd + kd].reshape(t, kv_heads, d).contiguous()
        v = qkv[:, qd + kd:].reshape(t, kv_heads, d).contiguous()
        if cos is not None:
            qk_norm_rope_table_(q, k, qw, kw, cos, sin, eps)
        else:
            qk_norm_rope_(q, k, qw, kw, positions, freqs, eps)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, qw, kw = ctx.saved_tensors
        cos, sin, positions, freqs = ctx.angles
        q_heads, kv_heads, d, eps, q_dtype, k_dtype = ctx.meta
        t, qd, kd = qkv.shape[0], q_heads * d, kv_heads * d
        dqkv = torch.empty_like(qkv)
        _, _, dqw, dkw = qk_norm_rope_backward(
            qkv[:, :qd].view(t, q_heads, d), qkv[:, qd:qd + kd].view(t, kv_heads, d), qw, kw, dq, dk,
            positions=positions, freqs=freqs, cos=cos, sin=sin, eps=eps,
            out_q=dqkv[:, :qd].view(t, q_heads, d), out_k=dqkv[:, qd:qd + kd].view(t, kv_heads, d))
        dqkv[:, qd + kd:].copy_(dv.reshape(t, kd))
        return dqkv, None, None, None, dqw.to(q_dtype), dkw.to(k_dtype), None, None, None, None, None


def qkv_norm_rope_autograd(qkv, q_heads, kv_heads, head_dim, q_weight, k_weight, *, cos=None, sin=None, positions=None,
                           freqs=None, eps=1e-6):
    """(q', k', v) [T, heads, D] from the stacked projection output, recording one backward for all three."""
    if cos is not None:
        cos, sin = cos.contiguous(), sin.contiguous()
    return _QkvNormRope.apply(qkv, q_heads, kv_heads, head_dim, q_weight, k_weight, cos, sin, positions, freqs, eps)


def qk_norm_rope_table_autograd(q, k, q_weight, k_weight, cos, sin, eps=1e-6):
    """(q', k') = QK-norm + RoPE of q [T,Hq,D], k [T,Hkv,D] (not in place), recording the backward."""
    return _QkNormRope.apply(q, k, q_weight, k_weight, cos.contiguous(), sin.contiguous(), None, None, eps)


def qk_norm_rope_autograd(q, k, q_weight, k_weight, positions, freqs, eps=1e-6):
    """As qk_norm_rope_table_autograd with the angles positions * inv_freq computed in the kernels."""
    return _QkNormRope.apply(q, k, q_weight, k_weight, None, None, positions, freqs, eps)


def linear_autograd(x, weight):
    """linear() that records its backward."""
    return _Linear.apply(x, weight)


def linear_geglu_autograd(x, gate_up):
    """linear_geglu() that records its backward."""
    return _LinearGeglu.apply(x, gate_up)


# --------------------------------------------------------------------------------------
# packed variable-length attention
# --------------------------------------------------------------------------------------

@dataclass
class AttentionPlan:
    """Device-side description of one pack for bg_varlen_attention: query tiles (heaviest
    first) and every token's own-key range.  Built once per pack and window, shared by all
    layers with that window."""

    tiles: torch.Tensor      # int32 [n_tiles, 8]
    row_lo: torch.Tensor     # int32 [T]
    row_hi: torch.Tensor     # int32 [T]
    tokens: int
    n_tiles: int
    pairs: int               # visible (query, key) pairs, for FLOP accounting
    tile_rows: int = 128     # query rows (tokens x GQA group) a tile may hold
    kv_tiles: torch.Tensor = None    # int32 [n_kv_tiles, 8], key tiles of the backward passes (optional)
    n_kv_tiles: int = 0
    own_extent: int = 0      # one past the last own-key row any tile addresses (host copy, for bounds checks)
    state_extent: int = 0    # one past the last state row any tile addresses
    pair_tiles: torch.Tensor = None  # int32 [n_pair_tiles, 8]: 256-row tiles served by CTA pairs (head_dim 256)
    n_pair_tiles: int = 0


def plan_rows(lengths, window, *, decoder):
    """Own-key range [lo, hi) of every packed token (numpy int64).

    Encoder: the segment, clipped to the bidirectional window with the odd-width rule
    (key visible iff 0 <= d < (w+1)//2 or 0 < -d < w//2+1, d = query - key position;
    bongard/packing.py:131-133).  Decoder: causal, optionally windowed (0 <= d < w;
    bongard/packing.py:122-125)."""
    lengths = np.asarray(lengths, dtype=np.int64)
    ends = np.cumsum(lengths)
    starts = ends - lengths
    seg_start = np.repeat(starts, lengths)
    seg_end = np.repeat(ends, lengths)
    t = np.arange(int(ends[-1]) if len(ends) else 0, dtype=np.int64)
    if decoder:
        lo = seg_start if window is None else np.maximum(seg_start, t - window + 1)
        hi = t + 1
    elif window is None:
        lo, hi = seg_start, seg_end
    else:
        lo = np.maximum(seg_start, t - (window + 1) // 2 + 1)
        hi = np.minimum(seg_end, t + window // 2 + 1)
    return lo, hi


@dataclass
class HostPlan:
    """Host half of an attention plan: one int32 array [tiles*8 | pair tiles*8 | row_lo | row_hi | key tiles*8]."""

    packed: np.ndarray
    tokens: int
    n_tiles: int
    pairs: int
    tile_rows: int = 128
    n_kv_tiles: int = 0      # key tiles for the backward passes, appended after row_hi
    own_extent: int = 0      # one past the last own-key row / state row the tiles address
    state_extent: int = 0
    n_pair_tiles: int = 0    # 256-row tiles for the CTA-pair kernel, stored after the 128-row tiles

    def to(self, device):
        dev = torch.from_numpy(self.packed).to(device, non_blocking=True)
        return self.view(dev)

    def padded(self, tokens, n_tiles):
        """The same plan in arrays of a fixed size (for launches captured in a CUDA graph): tiles
        beyond the plan's own are empty (no rows, no keys: the kernel skips them) and tokens
        beyond its own see no key."""
        if tokens < self.tokens or n_tiles < self.n_tiles:
            raise ValueError(f'plan of {self.tokens} tokens / {self.n_tiles} tiles does not fit {tokens} / {n_tiles}')
        if self.n_pair_tiles:
            raise ValueError('fixed-size plans hold 128-row tiles only (build the plan with pair=False)')
        n8, t = self.n_tiles * 8, self.tokens
        out = np.zeros(n_tiles * 8 + 2 * tokens, dtype=np.int32)
        out[:n8] = self.packed[:n8]
        out[n_tiles * 8:n_tiles * 8 + t] = self.packed[n8:n8 + t]
        out[n_tiles * 8 + tokens:n_tiles * 8 + tokens + t] = self.packed[n8 + t:n8 + 2 * t]
        return HostPlan(out, tokens, n_tiles, self.pairs, self.tile_rows, 0, self.own_extent, self.state_extent)

    def view(self, dev):
        s8, t = self.n_tiles * 8, self.tokens
        n8 = s8 + self.n_pair_tiles * 8
        plan = AttentionPlan(dev[:s8].view(-1, 8), dev[n8:n8 + t], dev[n8 + t:n8 + 2 * t], t, self.n_tiles, self.pairs,
                             self.tile_rows, own_extent=self.own_extent, state_extent=self.state_extent)
        if self.n_pair_tiles:
            plan.pair_tiles, plan.n_pair_tiles = dev[s8:n8].view(-1, 8), self.n_pair_tiles
        if self.n_kv_tiles:
            plan.kv_tiles = dev[n8 + 2 * t:n8 + 2 * t + self.n_kv_tiles * 8].view(-1, 8)
            plan.n_kv_tiles = self.n_kv_tiles
        return plan


PAIR_ATTENTION = False   # head_dim 256, forward-only plans: also cut runs into 256-row tiles for the CTA-pair kernel


def tile_rows(head_dim, pair=False):
    """Query rows (tokens x GQA group) one attention tile holds for a head size, as the library reports it:
    128 for the single-CTA kernel and the backward passes, 256 for the CTA-pair forward kernel (head_dim 256)."""
    if not head_dim:
        return 128
    lib = _lib.load()
    rows = lib.bg_attention_pair_tile_rows(int(head_dim)) if pair else 0
    return rows or lib.bg_attention_tile_rows(int(head_dim))


def _state_bank(owners, state_lengths, state_offsets):
    """Validated (offsets, lengths) of the state bank: `state_lengths[o]` rows starting at
    `state_offsets[o]` (default: the states lie back to back) for every owner o."""
    state_lengths = [int(n) for n in state_lengths]
    if any(n < 0 for n in state_lengths):
        raise ValueError('state lengths must not be negative')
    if state_offsets is None:
        state_offsets = np.concatenate(([0], np.cumsum(np.asarray(state_lengths, dtype=np.int64))))[:-1]
    state_offsets = [int(o) for o in state_offsets]
    if len(state_offsets) != len(state_lengths) or any(o < 0 for o in state_offsets):
        raise ValueError('state offsets must be one non-negative row per state')
    if any(not 0 <= int(o) < len(state_lengths) for o in owners):
        raise ValueError('an owner names a state that is not in the bank')
    return state_offsets, state_lengths


def make_host_kv_tiles(lengths, window, *, owners=None, state_lengths=None, state_offsets=None, keys_per_tile=128):
    """Key tiles for the backward passes (host arithmetic on lengths only): int32 [n, 8] rows
    {k_start, k_count, q_lo, q_hi, is_state, 0, 0, 0}.

    An own-key tile holds up to 128 consecutive keys of one segment; [q_lo, q_hi) are the query
    tokens whose key range meets it (which of them see which key is decided per pair from the
    row ranges).  A state tile holds keys of one owner's state; its queries are all tokens of the
    owner's questions, which therefore have to be consecutive in the pack.  Heaviest first."""
    lengths = [int(n) for n in lengths]
    decoder = owners is not None
    lo, hi = plan_rows(lengths, window, decoder=decoder)
    tiles = []
    offset = 0
    for n in lengths:
        if n:
            seg_lo, seg_hi = lo[offset:offset + n], hi[offset:offset + n]
            for k0 in range(offset, offset + n, keys_per_tile):
                count = min(keys_per_tile, offset + n - k0)
                q_lo = offset + int(np.searchsorted(seg_hi, k0, side='right'))       # first token with hi > k0
                q_hi = offset + int(np.searchsorted(seg_lo, k0 + count, side='left'))  # first token with lo >= end
                tiles.append((k0, count, q_lo, max(q_lo, q_hi), 0))
        offset += n
    if decoder:
        state_offsets, state_lengths = _state_bank(owners, state_lengths, state_offsets)
        runs, offset = [], 0
        for n, owner in zip(lengths, owners):
            if n:
                if runs and runs[-1][2] == owner:
                    runs[-1][1] = offset + n
                else:
                    runs.append([offset, offset + n, owner])
            offset += n
        seen = set()
        for start, end, owner in runs:
            if owner in seen:
                raise ValueError('the questions of one owner must be consecutive in the pack (backward pass)')
            seen.add(owner)
            base, length = int(state_offsets[owner]), int(state_lengths[owner])
            for k0 in range(0, length, keys_per_tile):
                tiles.append((base + k0, min(keys_per_tile, length - k0), start, end, 1))
    if not tiles:
        return np.zeros((0, 8), dtype=np.int32)
    out = np.zeros((len(tiles), 8), dtype=np.int32)
    out[:, :5] = np.asarray(tiles, dtype=np.int64)
    return out[np.argsort(-(out[:, 3] - out[:, 2]), kind='stable')]


def make_host_plan(lengths, window, *, group, owners=None, state_lengths=None, head_dim=None, backward=False,
                   state_offsets=None, pair=None):
    """Tile a pack of segments for the attention kernel (host arithmetic on lengths only).

    Encoder (owners None): tiles never cross a segment.  Decoder: consecutive questions of the
    same owner form one run; a tile is up to 128/group consecutive tokens of a run, so
    questions that share a state also share its key stream.  `state_offsets[o]` is the first row
    of owner o's state in the bank (default: states back to back in owner order).  Tiles are
    ordered heaviest first.  `pair` (default: PAIR_ATTENTION for forward-only plans) asks for the
    256-row tiles of the CTA-pair kernel where the head size has one."""
    lengths = [int(n) for n in lengths]
    if any(n < 0 for n in lengths):
        raise ValueError('segment lengths must not be negative')
    decoder = owners is not None
    if decoder and (state_lengths is None or len(owners) != len(lengths)):
        raise ValueError('decoder plans need state_lengths and one owner per segment')
    lo, hi = plan_rows(lengths, window, decoder=decoder)
    total = len(lo)
    single_rows = tile_rows(head_dim)
    pair_rows = tile_rows(head_dim, pair=True) if (PAIR_ATTENTION if pair is None else pair) and not backward else 0
    if pair_rows == single_rows:
        pair_rows = 0                       # this head size has no pair kernel
    runs = []      # [start, end, prefix_start, prefix_len, owner]
    offset = 0
    if decoder:
        state_offsets, state_lengths = _state_bank(owners, state_lengths, state_offsets)
        for n, owner in zip(lengths, owners):
            if runs and runs[-1][4] == owner:
                runs[-1][1] = offset + n
            else:
                runs.append([offset, offset + n, int(state_offsets[owner]), int(state_lengths[owner]), owner])
            offset += n
    else:
        for n in lengths:
            runs.append([offset, offset + n, 0, 0, -1])
            offset += n
    runs = [r for r in runs if r[1] > r[0]]
    if not runs:
        return HostPlan(np.zeros(0, dtype=np.int32), 0, 0, 0, single_rows)
    run = np.asarray([r[:4] for r in runs], dtype=np.int64)

    def tile(rows, part):
        """Tile records of `rows`-row tiles over the runs `part` ([start, end, prefix_start, prefix_len] each)."""
        part = part[part[:, 1] > part[:, 0]]
        if not len(part):
            return np.zeros((0, 8), dtype=np.int32)
        tq = rows // group
        big = np.int64(1) << 40
        counts = (part[:, 1] - part[:, 0] + tq - 1) // tq
        which = np.repeat(np.arange(len(part)), counts)
        first = np.cumsum(counts) - counts
        q_start = part[which, 0] + (np.arange(int(counts.sum())) - first[which]) * tq
        q_count = np.minimum(part[which, 1] - q_start, tq)
        # per-tile extremes of the rows' key ranges (reduceat over [q_start, q_start + q_count))
        edges = np.stack([q_start, q_start + q_count], axis=1).reshape(-1)      # index `total` is the pad element
        own_lo = np.minimum.reduceat(np.append(lo, big), edges)[::2]
        own_hi = np.maximum.reduceat(np.append(hi, -big), edges)[::2]
        lo_max = np.maximum.reduceat(np.append(lo, -big), edges)[::2]
        hi_min = np.minimum.reduceat(np.append(hi, big), edges)[::2]
        records = np.stack([q_start, q_count, own_lo, own_hi, lo_max, hi_min, part[which, 2], part[which, 3]], axis=1)
        work = part[which, 3] + own_hi - own_lo
        return records[np.argsort(-work, kind='stable')].astype(np.int32)

    if pair_rows:
        # A pair occupies two SMs for the whole key stream of its tile however few rows its second CTA holds.  So a run
        # is cut into full 256-row tiles, and what is left goes to a pair only if it fills more than one CTA; a
        # shorter rest becomes one 128-row tile for the single-CTA kernel.  The cut depends on the run alone.
        tqp, tqs = pair_rows // group, single_rows // group
        n = run[:, 1] - run[:, 0]
        rest = n % tqp
        pair_tokens = np.where(rest > tqs, n, n - rest) if pair is None else n      # pair=True: everything on pairs
        pair_part = np.stack([run[:, 0], run[:, 0] + pair_tokens, run[:, 2], run[:, 3]], axis=1)
        single_part = np.stack([run[:, 0] + pair_tokens, run[:, 1], run[:, 2], run[:, 3]], axis=1)
        pair_tiles, tiles = tile(pair_rows, pair_part), tile(single_rows, single_part)
    else:
        pair_tiles, tiles = np.zeros((0, 8), dtype=np.int32), tile(single_rows, run)
    rows = single_rows
    parts = [tiles.reshape(-1), pair_tiles.reshape(-1), lo.astype(np.int32), hi.astype(np.int32)]
    n_kv = 0
    if backward:
        kv = make_host_kv_tiles(lengths, window, owners=owners, state_lengths=state_lengths, state_offsets=state_offsets)
        parts.append(kv.reshape(-1))
        n_kv = kv.shape[0]
    pairs = int((hi - lo).sum())
    if decoder:
        pairs += int(sum(n * state_lengths[o] for n, o in zip(lengths, owners)))
    state_extent = int((run[:, 2] + run[:, 3])[run[:, 3] > 0].max(initial=0))
    return HostPlan(np.concatenate(parts), total, tiles.shape[0], pairs, rows, n_kv, total, state_extent,
                    pair_tiles.shape[0])


def make_plan(lengths, window, device, *, group, owners=None, state_lengths=None, head_dim=None, backward=False,
              state_offsets=None, pair=None):
    return make_host_plan(lengths, window, group=group, owners=owners, state_lengths=state_lengths,
                          head_dim=head_dim, backward=backward, state_offsets=state_offsets, pair=pair).to(device)


def check_plan_bounds(plan, key_rows, state_rows):
    """Host check that every key row a plan addresses exists: raises ValueError before any launch
    (the forward would read zero-filled rows, the backward would store state gradients past the
    end of their buffers)."""
    if plan.own_extent > key_rows:
        raise ValueError(f'the attention plan addresses own-key rows up to {plan.own_extent}, k/v hold {key_rows}')
    if plan.state_extent > state_rows:
        raise ValueError(f'the attention plan addresses state rows up to {plan.state_extent}, '
                         f'the state keys/values hold {state_rows}')


def varlen_attention(q, k, v, plan, scale, cross=None, return_lse=False):
    """q [T,Hq,D], k/v [T,Hkv,D] (token-strided views allowed), cross = (ck, cv) [S,Hkv,D].
    Returns out [T, Hq*D] (and lse [Hq,T] fp32)."""
    lib = _lib.load()
    for t, name in ((q, 'q'), (k, 'k'), (v, 'v')):
        _need(t, name)
        if t.ndim != 3 or t.stride(2) != 1:
            raise ValueError(f'{name} must be [T, heads, D] with a contiguous last dimension')
    if k.stride() != v.stride() or k.shape != v.shape:
        raise ValueError('k and v must share shape and strides')
    tq, hq, d = q.shape
    tk, hkv = k.shape[0], k.shape[1]
    if plan.tokens != tq:
        raise ValueError(f'plan was built for {plan.tokens} tokens, q has {tq}')
    if plan.tile_rows > lib.bg_attention_tile_rows(d):
        raise ValueError(f'plan has {plan.tile_rows}-row tiles; head_dim {d} takes {lib.bg_attention_tile_rows(d)}')
    if plan.n_pair_tiles and lib.bg_attention_pair_tile_rows(d) == 0:
        raise ValueError(f'plan has tiles for CTA pairs; head_dim {d} has no pair kernel')
    ck = cv = None
    ts = ldc = hsc = 0
    if cross is not None:
        ck, cv = cross
        _need(ck, 'cross keys'), _need(cv, 'cross values')
        if ck.shape != cv.shape or ck.stride() != cv.stride() or ck.shape[1:] != k.shape[1:] or ck.stride(2) != 1:
            raise ValueError('cross keys/values must be [S, kv_heads, D] with equal strides')
        ts, ldc, hsc = ck.shape[0], ck.stride(0), ck.stride(1)
    check_plan_bounds(plan, tk, ts)
    out = torch.empty((tq, hq * d), device=q.device, dtype=BF16)
    lse = torch.empty((hq, tq), device=q.device, dtype=torch.float32) if return_lse else None
    timer = ATTN_TIMER
    begin = timer.start() if timer is not None else None
    for entry, name, tiles, n_tiles in ((lib.bg_varlen_attention_pair, 'bg_varlen_attention_pair', plan.pair_tiles, plan.n_pair_tiles),
                                        (lib.bg_varlen_attention, 'bg_varlen_attention', plan.tiles, plan.n_tiles)):
        if n_tiles:       # the two kernels write disjoint rows of out / lse
            _lib.check(entry(
                _ptr(q), q.stride(0), q.stride(1), _ptr(k), _ptr(v), k.stride(0), k.stride(1), _ptr(ck), _ptr(cv), ldc, hsc,
                _ptr(out), _ptr(lse), _ptr(tiles), n_tiles, _ptr(plan.row_lo), _ptr(plan.row_hi), tq, tk, ts, hq, hkv, d,
                float(scale), _stream()), name)
    if timer is not None:
        timer.stop(begin, 4 * d * hq * plan.pairs)
    return (out, lse) if return_lse else out


def varlen_attention_backward(q, k, v, plan, scale, out, lse, dout, cross=None):
    """Gradients of varlen_attention: (dq, dk, dv) or (dq, dk, dv, dck, dcv) with a state prefix.
    `plan` must carry key tiles (make_plan(..., backward=True)); `out`, `lse` are the forward's
    results, `dout` [T, Hq*D] or [T, Hq, D] the gradient of `out`."""
    lib = _lib.load()
    for t, name in ((q, 'q'), (k, 'k'), (v, 'v'), (out, 'out'), (dout, 'dout')):
        _need(t, name)
    _need(lse, 'lse', torch.float32)
    tq, hq, d = q.shape
    tk, hkv = k.shape[0], k.shape[1]
    if plan.tokens != tq or plan.kv_tiles is None:
        raise ValueError('the plan must match q and carry key tiles (make_plan(..., backward=True))')
    if k.stride() != v.stride() or k.shape != v.shape:
        raise ValueError('k and v must share shape and strides')
    out = out.reshape(tq, hq * d)
    if not out.is_contiguous() or not lse.is_contiguous() or lse.shape != (hq, tq):
        raise ValueError('out must be contiguous [T, Hq*D] and lse contiguous [Hq, T]')
    dout = dout.reshape(tq, hq, d)
    if dout.stride(2) != 1:
        dout = dout.contiguous()
    ck = cv = dck = dcv = None
    ts = ldc = hsc = 0
    if cross is not None:
        ck, cv = cross
        _need(ck, 'cross keys'), _need(cv, 'cross values')
        if ck.shape != cv.shape or ck.stride() != cv.stride() or ck.shape[1:] != k.shape[1:] or ck.stride(2) != 1:
            raise ValueError('cross keys/values must be [S, kv_heads, D] with equal strides')
        ts, ldc, hsc = ck.shape[0], ck.stride(0), ck.stride(1)
    check_plan_bounds(plan, tk, ts)
    if cross is not None:
        dck = torch.zeros((ts, hkv, d), device=q.device, dtype=BF16)    # states without a question keep zero
        dcv = torch.zeros((ts, hkv, d), device=q.device, dtype=BF16)
    dq = torch.empty((tq, hq, d), device=q.device, dtype=BF16)
    dk = torch.empty((tk, hkv, d), device=q.device, dtype=BF16)
    dv = torch.empty((tk, hkv, d), device=q.device, dtype=BF16)
    delta = torch.empty((hq, tq), device=q.device, dtype=torch.float32)
    _lib.check(lib.bg_varlen_attention_backward(
        _ptr(q), q.stride(0), q.stride(1), _ptr(k), _ptr(v), k.stride(0), k.stride(1), _ptr(ck), _ptr(cv), ldc, hsc,
        _ptr(out), _ptr(dout), dout.stride(0), dout.stride(1), _ptr(lse), _ptr(delta), _ptr(dq), _ptr(dk), _ptr(dv),
        _ptr(dck), _ptr(dcv), _ptr(plan.tiles), plan.n_tiles, _ptr(plan.kv_tiles), plan.n_kv_tiles,
        _ptr(plan.row_lo), _ptr(plan.row_hi), tq, tk, ts, hq, hkv, d, float(scale), _stream()),
        'bg_varlen_attention_backward')
    return (dq, dk, dv) if cross is None else (dq, dk, dv, dck, dcv)


class _VarlenAttention(torch.autograd.Function):
    """out = varlen_attention(q, k, v[, state k, v]) with the tensor-core backward."""

    @staticmethod
    def forward(ctx, q, k, v, ck, cv, plan, scale):
        cross = None if ck is None else (ck, cv)
        out, lse = varlen_attention(q, k, v, plan, scale, cross, return_lse=True)
        ctx.save_for_backward(q, k, v, ck, cv, out, lse)
        ctx.plan, ctx.scale = plan, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, ck, cv, out, lse = ctx.saved_tensors
        cross = None if ck is None else (ck, cv)
        grads = varlen_attention_backward(q, k, v, ctx.plan, ctx.scale, out, lse, dout, cross)
        dq, dk, dv = grads[:3]
        dck, dcv = (grads[3], grads[4]) if cross is not None else (None, None)
        return dq, dk, dv, dck, dcv, None, None


def varlen_attention_autograd(q, k, v, plan, scale, cross=None):
    """varlen_attention that records its backward (plan built with backward=True)."""
    ck, cv = cross if cross is not None else (None, None)
    return _VarlenAttention.apply(q, k, v, ck, cv, plan, scale)


# --------------------------------------------------------------------------------------
# judgment head
# --------------------------------------------------------------------------------------

def judgment_head(hidden, cand_rows, dec_rows, w, candidate, global_readout):
    lib = _lib.load()
    _need(hidden, 'hidden'), _need(cand_rows, 'cand_rows', torch.int32), _need(dec_rows, 'dec_rows', torch.int32)
    for t in (w, candidate, global_readout):
        _need(t, 'head weight')
        if not t.is_contiguous():
            raise ValueError('head weights must be contiguous')
    n = cand_rows.numel()
    logits = torch.empty(n, device=hidden.device, dtype=torch.float32)
    _lib.check(lib.bg_judgment_head(_ptr(hidden), hidden.stride(0), _ptr(cand_rows), _ptr(dec_rows), _ptr(w),
                                    _ptr(candidate), _ptr(global_readout), _ptr(logits), n, hidden.shape[1],
                                    candidate.shape[0], _stream()), 'bg_judgment_head')
    return logits


def candidate_softmax(logits, offsets, temperature=1.0):
    """Per-question float64 probabilities; question i owns logits[offsets[i]:offsets[i+1]]."""
    lib = _lib.load()
    _need(logits, 'logits', torch.float32), _need(offsets, 'offsets', torch.int32)
    probs = torch.empty(logits.numel(), device=logits.device, dtype=torch.float64)
    _lib.check(lib.bg_candidate_softmax(_ptr(logits), _ptr(offsets), _ptr(probs), offsets.numel() - 1,
                                        float(temperature), _stream()), 'bg_candidate_softmax')
    return probs


# --------------------------------------------------------------------------------------
# FP8 E4M3 with per-128 block scales
# --------------------------------------------------------------------------------------

@dataclass
class Fp8Weight:
    """A weight quantised once: E4M3 values [N, K] (uint8 storage) and inverse scales per 128 x 128 tile."""

    q: torch.Tensor
    inv_scale: torch.Tensor
    shape: tuple


def quantize_rows(x):
    """1 x 128 dynamic quantisation of x [M, K] -> (q uint8 [M, K], inverse scales fp32 [K/128, M])."""
    lib = _lib.load()
    flat, m, k, ldx = _rows(x, 'x')
    q = torch.empty((m, k), device=x.device, dtype=torch.uint8)
    inv = torch.empty((k // 128, m), device=x.device, dtype=torch.float32)
    _lib.check(lib.bg_quantize_e4m3_rows(_ptr(flat), ldx, _ptr(q), k, _ptr(inv), m, k, _stream()),
               'bg_quantize_e4m3_rows')
    return q, inv


def quantize_weight(weight):
    """128 x 128 dynamic quantisation of a [N, K] weight."""
    lib = _lib.load()
    _need(weight, 'weight')
    if weight.ndim != 2 or weight.stride(1) != 1:
        raise ValueError('weight must be [N, K] with contiguous rows')
    n, k = weight.shape
    q = torch.empty((n, k), device=weight.device, dtype=torch.uint8)
    inv = torch.empty(((n + 127) // 128, k // 128), device=weight.device, dtype=torch.float32)
    _lib.check(lib.bg_quantize_e4m3_tiles(_ptr(weight), weight.stride(0), _ptr(q), k, _ptr(inv), n, k, _stream()),
               'bg_quantize_e4m3_tiles')
    return Fp8Weight(q, inv, (n, k))


_WORKSPACE = {}


_RETIRED_WORKSPACES = []


def _workspace(device, nbytes):
    """Scratch for the quantised activations of bg_linear_fp8: one grow-only buffer per device.

    While a CUDA graph is being captured the scratch is allocated per call instead, so that it comes
    from the graph's private pool and lives as long as the graph: a captured kernel keeps the address
    it was given, and a shared buffer that later grew (and was replaced) would leave earlier graphs
    writing into memory the allocator has handed to someone else.  For the same reason a buffer that
    is outgrown in eager mode is retired, not freed: a graph captured by other means may still name it."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(max(nbytes, 1), device=device, dtype=torch.uint8)
    buf = _WORKSPACE.get(device)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _RETIRED_WORKSPACES.append(buf)
        buf = torch.empty(max(nbytes, 1 << 20), device=device, dtype=torch.uint8)
        _WORKSPACE[device] = buf
    return buf


def linear_fp8(x, weight: Fp8Weight, *, geglu=False):
    """bf16 x [..., K] times an Fp8Weight: dynamic 1 x 128 activation scales, E4M3 tensor-core
    contraction, fp32 accumulation, bf16 result.  geglu=True treats the weight as [gate; up]."""
    lib = _lib.load()
    flat, m, k, ldx = _rows(x, 'x')
    rows, wk = weight.shape
    if wk != k:
        raise ValueError(f'weight has K={wk}, input has {k}')
    n = rows // 2 if geglu else rows
    out = torch.empty((m, n), device=x.device, dtype=BF16)
    need = lib.bg_linear_fp8_workspace_bytes(m, k)
    ws = _workspace(x.device, need)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    _lib.check(lib.bg_linear_fp8(_ptr(flat), ldx, _ptr(weight.q), k, _ptr(weight.inv_scale), _ptr(out), n, m, n, k,
                                 1 if geglu else 0, _ptr(ws), ws.numel(), _stream()), 'bg_linear_fp8')
    if timer is not None:
        timer.stop(begin, (4 if geglu else 2) * m * n * k)
    return out.view(*x.shape[:-1], n)


def gemm_fp8(aq, a_inv_t, weight: Fp8Weight, *, geglu=False):
    """Pre-quantised activations (from quantize_rows) times an Fp8Weight."""
    lib = _lib.load()
    m, k = aq.shape
    rows = weight.shape[0]
    n = rows // 2 if geglu else rows
    out = torch.empty((m, n), device=aq.device, dtype=BF16)
    _lib.check(lib.bg_gemm_fp8_block128(_ptr(aq), k, _ptr(a_inv_t), _ptr(weight.q), k, _ptr(weight.inv_scale),
                                        _ptr(out), n, m, n, k, 1 if geglu else 0, _stream()), 'bg_gemm_fp8_block128')
    return out


@dataclass
class Mxfp8Tensor:
    """E4M3 values [rows, K] with UE8M0 scales per 32 K elements in the 512-byte atom layout."""

    q: torch.Tensor            # uint8 [rows, K]
    scales: torch.Tensor       # uint8 [ceil(rows/128) * K/128 * 512]

    @property
    def shape(self):
        return self.q.shape


def quantize_mxfp8(x):
    """bf16 [rows, K] -> Mxfp8Tensor (K a multiple of 128)."""
    lib = _lib.load()
    flat, m, k, ldx = _rows(x, 'x')
    q = torch.empty((m, k), device=x.device, dtype=torch.uint8)
    scales = torch.zeros(lib.bg_mxfp8_scale_bytes(m, k), device=x.device, dtype=torch.uint8)
    _lib.check(lib.bg_quantize_mxfp8(_ptr(flat), ldx, _ptr(q), k, _ptr(scales), m, k, _stream()), 'bg_quantize_mxfp8')
    return Mxfp8Tensor(q, scales)


def gemm_mxfp8(a: Mxfp8Tensor, weight: Mxfp8Tensor, *, geglu=False):
    """Quantised activations times quantised weights: [m, K] x [N, K]^T -> bf16 [m, N] (N/2 with GeGLU)."""
    lib = _lib.load()
    m, k = a.shape
    rows = weight.shape[0]
    if weight.shape[1] != k:
        raise ValueError(f'weight has K={weight.shape[1]}, input has {k}')
    n = rows // 2 if geglu else rows
    out = torch.empty((m, n), device=a.q.device, dtype=BF16)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    _lib.check(lib.bg_gemm_mxfp8(_ptr(a.q), k, _ptr(a.scales), _ptr(weight.q), k, _ptr(weight.scales), _ptr(out), n,
                                 m, n, k, 1 if geglu else 0, _stream()), 'bg_gemm_mxfp8')
    if timer is not None:
        timer.stop(begin, (4 if geglu else 2) * m * n * k)
    return out


def _mx_empty(rows, k, device):
    lib = _lib.load()
    return Mxfp8Tensor(torch.empty((rows, k), device=device, dtype=torch.uint8),
                       torch.zeros(lib.bg_mxfp8_scale_bytes(rows, k), device=device, dtype=torch.uint8))


def rmsnorm_mxfp8(x, weight, eps=1e-6):
    """rmsnorm(x) * (1 + weight) written as MXFP8 for the GEMM that consumes it."""
    lib = _lib.load()
    flat, rows, h, ldx = _rows(x, 'x')
    out = _mx_empty(rows, h, x.device)
    _lib.check(lib.bg_rmsnorm_mxfp8(_ptr(flat), ldx, _ptr(_need(weight, 'weight')), _ptr(out.q), _ptr(out.scales), rows,
                                    h, eps, _stream()), 'bg_rmsnorm_mxfp8')
    return out


def add_rmsnorm_mxfp8_(y, w_post, resid, w_next, eps=1e-6):
    """add_rmsnorm_ whose normalised output is MXFP8."""
    lib = _lib.load()
    _need(y, 'y'), _need(resid, 'resid')
    if not (y.is_contiguous() and resid.is_contiguous()) or y.shape != resid.shape:
        raise ValueError('y and resid must be contiguous and of equal shape')
    h = y.shape[-1]
    rows = y.numel() // h
    out = _mx_empty(rows, h, y.device)
    _lib.check(lib.bg_add_rmsnorm_mxfp8(_ptr(y), _ptr(_need(w_post, 'w_post')), _ptr(resid), _ptr(_need(w_next, 'w_next')),
                                        _ptr(out.q), _ptr(out.scales), rows, h, eps, _stream()), 'bg_add_rmsnorm_mxfp8')
    return out


def gemm_mxfp8_geglu_q(a: Mxfp8Tensor, gate_up: Mxfp8Tensor):
    """gelu_tanh(a gate^T) * (a up^T) written directly as MXFP8 for the down projection."""
    lib = _lib.load()
    m, k = a.shape
    n = gate_up.shape[0] // 2
    if gate_up.shape[1] != k:
        raise ValueError(f'weight has K={gate_up.shape[1]}, input has {k}')
    q = torch.empty((m, n), device=a.q.device, dtype=torch.uint8)
    scales = torch.zeros(lib.bg_mxfp8_scale_bytes(m, n), device=a.q.device, dtype=torch.uint8)
    timer = GEMM_TIMER
    begin = timer.start() if timer is not None else None
    _lib.check(lib.bg_gemm_mxfp8_geglu_q(_ptr(a.q), k, _ptr(a.scales), _ptr(gate_up.q), k, _ptr(gate_up.scales), _ptr(q),
                                         n, _ptr(scales), m, n, k, _stream()), 'bg_gemm_mxfp8_geglu_q')
    if timer is not None:
        timer.stop(begin, 4 * m * n * k)
    return Mxfp8Tensor(q, scales)


def mlp_mxfp8(x, gate_up: Mxfp8Tensor, down: Mxfp8Tensor):
    """The gated MLP on MXFP8 weights: quantise x, gate|up GEMM with the GeGLU epilogue emitting MXFP8,
    down GEMM.  The hidden activation never exists in bf16."""
    if isinstance(x, Mxfp8Tensor):
        return gemm_mxfp8(gemm_mxfp8_geglu_q(x, gate_up), down)
    flat, m, k, _ = _rows(x, 'x')
    out = gemm_mxfp8(gemm_mxfp8_geglu_q(quantize_mxfp8(flat), gate_up), down)
    return out.view(*x.shape[:-1], out.shape[-1])


def linear_mxfp8(x, weight: Mxfp8Tensor, *, geglu=False):
    """bf16 x [..., K] times an MXFP8 weight: dynamic 1 x 32 power-of-two activation scales, block-scaled
    tensor-core contraction, bf16 result."""
    if isinstance(x, Mxfp8Tensor):
        return gemm_mxfp8(x, weight, geglu=geglu)
    out = gemm_mxfp8(quantize_mxfp8(x), weight, geglu=geglu)
    return out.view(*x.shape[:-1], out.shape[-1])


def linear_fp8_static(x, weight: Fp8Weight, *, geglu=False):
    """linear_fp8 without any scratch allocation: the quantised activations live in a fixed
    buffer inside the library (see bg_linear_fp8_static).  Raises B200Error when the activation
    does not fit that buffer."""
    lib = _lib.load()
    flat, m, k, ldx = _rows(x, 'x')
    rows, wk = weight.shape
    if wk != k:
        raise ValueError(f'weight has K={wk}, input has {k}')
    n = rows // 2 if geglu else rows
    out = torch.empty((m, n), device=x.device, dtype=BF16)
    _lib.check(lib.bg_linear_fp8_static(_ptr(flat), ldx, _ptr(weight.q), k, _ptr(weight.inv_scale), _ptr(out), n, m, n,
                                        k, 1 if geglu else 0, _stream()), 'bg_linear_fp8_static')
    return out.view(*x.shape[:-1], n)
