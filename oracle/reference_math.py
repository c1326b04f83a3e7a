"""CPU restatement of the reference's transformer inference hot path.  TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA path, never the product: only tests, the
smoke check and the benchmark's CPU-baseline leg may import it.  Nothing in the
package imports it, and the package has no CPU fallback.

Every function restates, op for op, what the reference computes on its
``device="cpu"`` path, in plain PyTorch CPU arithmetic in the dtype of its
inputs (fp32 is the ground truth; bf16 reproduces the reference's own rounding
points).  Part of that arithmetic lives in a third-party dependency that is not
vendored with the reference (``transformers`` T5Gemma2, pinned ==5.17.0 in the
reference's pyproject.toml:16); those functions restate its published model
code and cite it as ``HF:`` (models/t5gemma2/modeling_t5gemma2.py, line numbers
of release 5.5.0).

Parity pin: the reference ships no tests, golden vectors or fixtures for this
path, so the restatement is pinned against the reference itself, imported and
run on CPU next to the checkout (tests/golden/make_golden.py writes the
fixtures; tests/test_oracle_golden.py replays them without the reference).
The FP8 block-scaled functions have no runnable reference counterpart (its FP8
linears need torchao, absent offline, and serve plain bf16 in eval mode), so
for those parity is unpinned: they restate the dynamic-amax scaling rule only.
"""

from __future__ import annotations

import math

import torch
from torch.nn import functional as F

E4M3_MAX = 448.0


# --------------------------------------------------------------------------------------
# glue: RMSNorm, embedding, rotary tables
# --------------------------------------------------------------------------------------

def rmsnorm(x, weight, eps=1e-6):
    """HF:61-69 T5Gemma2RMSNorm: fp32 math, (1 + w) multiplied before the cast back
    (the rule bongard/mps_inference.py:78-82 documents)."""
    xf = x.float()
    out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    out = out * (1.0 + weight.float())
    return out.type_as(x)


def embed(ids, table, eoi_embedding, hidden, eoi_token=256_000):
    """HF:644-647 scaled word embedding: rows times sqrt(hidden) rounded to the weight
    dtype; rows of the end-of-image token are replaced by a separate vector."""
    scale = torch.tensor(math.sqrt(hidden)).to(table.dtype)
    out = table[ids] * scale
    out[ids == eoi_token] = eoi_embedding.to(out.dtype)
    return out


def rope_tables(positions, head_dim, theta, dtype):
    """HF:132-172 default rotary embedding: inv_freq = theta^(-2i/D) in fp32, angles
    = position * inv_freq, cos/sin of cat(angles, angles), cast to the activation dtype."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    freqs = positions.float()[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps=1e-6):
    """bongard/attention.py:172-180 project_qk after the projections: per-head RMSNorm
    (HF:61-69), then rotate-half RoPE (HF:175-205) in the activation dtype.
    q [T,Hq,D], k [T,Hkv,D], cos/sin [T,D].  cos=None skips the rotation, which is how
    the decoder's shared state keys are made (bongard/model.py:135-139)."""
    q, k = rmsnorm(q, q_weight, eps), rmsnorm(k, k_weight, eps)
    if cos is None:
        return q, k
    c, s = cos[:, None, :], sin[:, None, :]
    return (q * c) + (rotate_half(q) * s), (k * c) + (rotate_half(k) * s)


# --------------------------------------------------------------------------------------
# packed variable-length attention
# --------------------------------------------------------------------------------------

def encoder_visible(distance, window):
    """bongard/packing.py:131-133 (HF:737-753): bidirectional window with the odd-width
    rule; distance = query position - key position inside one segment."""
    if window is None:
        return torch.ones_like(distance, dtype=torch.bool)
    return (distance < (window + 1) // 2) & (-distance < window // 2 + 1)


def decoder_visible(distance, window):
    """bongard/packing.py:122-125, bongard/attention.py:195-202: causal, optionally windowed."""
    visible = distance >= 0
    if window is not None:
        visible = visible & (distance < window)
    return visible


def _segment_attention(q, k, v, mask, scale):
    """q [L,Hq,D], k/v [Lk,Hkv,D], mask [L,Lk] -> out [L,Hq,D], lse [Hq,L] (natural log).
    Same arithmetic as F.scaled_dot_product_attention(enable_gqa=True) with a dense mask
    (bongard/packing.py:173-175), with the softmax kept in fp32."""
    hq, hkv = q.shape[1], k.shape[1]
    group = hq // hkv
    qf = q.float().permute(1, 0, 2)                                  # [Hq,L,D]
    kf = k.float().permute(1, 0, 2).repeat_interleave(group, 0)      # [Hq,Lk,D]
    vf = v.float().permute(1, 0, 2).repeat_interleave(group, 0)
    scores = torch.matmul(qf, kf.transpose(1, 2)) * scale
    scores = scores.masked_fill(~mask[None], -torch.inf)
    lse = torch.logsumexp(scores, dim=-1)
    p = torch.exp(scores - torch.where(torch.isfinite(lse), lse, 0.0)[..., None])
    out = torch.matmul(p, vf)
    return out.permute(1, 0, 2).to(q.dtype), lse


def varlen_attention(q, k, v, lengths, scale, window, *, cross=None, owners=None, state_lengths=None):
    """Packed attention over independent segments, segment by segment.

    Encoder (cross=None): bongard/flash_varlen.py:13-22 for an inactive window, the mask of
    bongard/packing.py:116-136 otherwise.  Decoder (cross=(ck, cv) [S_total,Hkv,D]): every
    question sees its owner's complete state plus its own causal (windowed) prefix under one
    softmax - the state-prefix rule of bongard/flash_varlen.py:1-8, 61-77 and the
    [own | state] key concatenation of bongard/packing.py:196-198.
    q [T,Hq,D]; k,v [T,Hkv,D].  Returns out [T,Hq,D], lse [Hq,T] fp32.
    """
    outs, lses, offset = [], [], 0
    state_offsets = None
    if cross is not None:
        state_offsets = [0]
        for s in state_lengths:
            state_offsets.append(state_offsets[-1] + s)
    for index, length in enumerate(lengths):
        rows = slice(offset, offset + length)
        pos = torch.arange(length)
        distance = pos[:, None] - pos[None, :]
        if cross is None:
            mask = encoder_visible(distance, window)
            ks, vs = k[rows], v[rows]
        else:
            owner = owners[index]
            srows = slice(state_offsets[owner], state_offsets[owner + 1])
            ns = state_lengths[owner]
            mask = torch.cat((torch.ones(length, ns, dtype=torch.bool), decoder_visible(distance, window)), 1)
            ks, vs = torch.cat((cross[0][srows], k[rows])), torch.cat((cross[1][srows], v[rows]))
        o, l = _segment_attention(q[rows], ks, vs, mask, scale)
        outs.append(o)
        lses.append(l)
        offset += length
    return torch.cat(outs), torch.cat(lses, dim=1)


def merge_partitions(parts):
    """bongard/attention.py:166-169: softmax over partition LSEs weights their outputs."""
    outputs, lses = zip(*parts)
    weights = torch.stack(lses).softmax(0)
    return (torch.stack(outputs) * weights.unsqueeze(-1)).sum(0)


# --------------------------------------------------------------------------------------
# linears and the gated MLP
# --------------------------------------------------------------------------------------

def linear(x, weight):
    """F.linear without bias: what TELinear / TrainingLinear serve in eval mode
    (bongard/te_linear.py:61-62, bongard/float8_training.py:20-21)."""
    return F.linear(x, weight)


def geglu_mlp(x, gate, up, down):
    """HF:87-91 T5Gemma2MLP with gelu_pytorch_tanh: down(gelu_tanh(gate x) * up x);
    the same contraction bongard/te_linear.py:98-103 fuses as gate_up -> GeGLU -> down."""
    return F.linear(F.gelu(F.linear(x, gate), approximate='tanh') * F.linear(x, up), down)


def quantize_e4m3_block(x, block_rows, block_cols):
    """Dynamic-amax E4M3 quantisation over (block_rows x block_cols) blocks.

    The scaling rule is the one the reference's FP8 linears apply per call
    (bongard/float8_training.py:35-44: dynamic, amax-derived scales, no history):
    scale = 448 / max(amax, 1e-12); values are clamped to +-448 and rounded to E4M3.
    Returns (q float8_e4m3fn, inverse scales fp32 [rows/block_rows, cols/block_cols]).
    Activations use 1 x 128 blocks, weights 128 x 128.
    """
    rows, cols = x.shape
    pr, pc = -rows % block_rows, -cols % block_cols
    xf = F.pad(x.float(), (0, pc, 0, pr))
    br, bc = xf.shape[0] // block_rows, xf.shape[1] // block_cols
    tiles = xf.reshape(br, block_rows, bc, block_cols)
    amax = tiles.abs().amax(dim=(1, 3))
    # tensor / tensor is an IEEE division (a python scalar divided by a tensor is reciprocal-multiply)
    scale = torch.full_like(amax, E4M3_MAX) / amax.clamp_min(1e-12)
    q = (tiles * scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX)
    q = q.reshape(xf.shape)[:rows, :cols].to(torch.float8_e4m3fn)
    return q, (torch.ones_like(scale) / scale).float()


def dequantize_block(q, inv_scale, block_rows, block_cols):
    rows, cols = q.shape
    s = inv_scale.repeat_interleave(block_rows, 0)[:rows].repeat_interleave(block_cols, 1)[:, :cols]
    return q.float() * s


def linear_fp8_block128(x, weight, out_dtype=torch.bfloat16):
    """E4M3 linear with 1x128 activation and 128x128 weight scales, fp32 accumulate."""
    xq, xs = quantize_e4m3_block(x, 1, 128)
    wq, ws = quantize_e4m3_block(weight, 128, 128)
    out = dequantize_block(xq, xs, 1, 128) @ dequantize_block(wq, ws, 128, 128).t()
    return out.to(out_dtype)


def geglu_mlp_fp8_block128(x, gate, up, down, out_dtype=torch.bfloat16):
    g = linear_fp8_block128(x, gate, out_dtype)
    u = linear_fp8_block128(x, up, out_dtype)
    return linear_fp8_block128(F.gelu(g, approximate='tanh') * u, down, out_dtype)


def quantize_mxfp8(x):
    """MXFP8 as the `mxfp8` recipe defines it (bongard/te_linear.py:32-39 -> Transformer Engine
    MXFP8BlockScaling; OCP Microscaling v1.0): per 32 consecutive K elements a power-of-two scale
    2^e with e = ceil(log2(amax / 448)) clamped to [-127, 127], values e4m3(x * 2^-e).
    Returns (values as float32 holding exact E4M3 numbers, exponents int32 [rows, K/32])."""
    rows, k = x.shape
    blocks = x.float().view(rows, k // 32, 32)
    amax = blocks.abs().amax(-1)
    mant, ex = torch.frexp(amax / 448.0)              # amax/448 = mant * 2^ex, mant in [0.5, 1)
    e = torch.where(mant == 0.5, ex - 1, ex)
    e = torch.where(amax > 0, e, torch.full_like(e, -127)).clamp(-127, 127)
    scaled = blocks * torch.exp2(-e.float())[..., None]
    q = scaled.to(torch.float8_e4m3fn).float()
    return q.view(rows, k), e.int()


def dequantize_mxfp8(q, e):
    rows, k = q.shape
    return (q.view(rows, k // 32, 32) * torch.exp2(e.float())[..., None]).view(rows, k)


def linear_mxfp8(x, weight, out_dtype=torch.bfloat16):
    """y = dq(x) dq(w)^T in fp32 (products of E4M3 values and powers of two are exact; only the
    accumulation order differs from the tensor core), rounded to the activation dtype."""
    xq, xe = quantize_mxfp8(x)
    wq, we = quantize_mxfp8(weight)
    return (dequantize_mxfp8(xq, xe) @ dequantize_mxfp8(wq, we).t()).to(out_dtype)


def geglu_mlp_mxfp8(x, gate, up, down, out_dtype=torch.bfloat16):
    """gate|up in fp32 accumulators -> gelu_tanh(g) * u -> activation dtype -> down, as the fused GEMM does."""
    xq, xe = quantize_mxfp8(x)
    xd = dequantize_mxfp8(xq, xe)
    g = xd @ dequantize_mxfp8(*quantize_mxfp8(gate)).t()
    u = xd @ dequantize_mxfp8(*quantize_mxfp8(up)).t()
    h = (F.gelu(g, approximate='tanh') * u).to(out_dtype)
    return linear_mxfp8(h, down, out_dtype)


# --------------------------------------------------------------------------------------
# judgment head and probabilities
# --------------------------------------------------------------------------------------

def judgment_head(h, g, w, candidate, global_readout):
    """bongard/model.py:92-95: w.h + (C h).(G g) / sqrt(256)."""
    return F.linear(h, w).squeeze(-1) + (F.linear(h, candidate) * F.linear(g, global_readout)).sum(-1) / math.sqrt(256)


def probabilities(logits, temperature=1.0):
    """bongard/inference.py:54-73: float64 temperature softmax, renormalised."""
    z = logits.detach().cpu().double()
    if temperature >= 1:
        z = z / temperature
        z = z - z.max()
    else:
        z = (z - z.max()) / temperature
    p = torch.softmax(z, dim=-1)
    return p / p.sum()


# --------------------------------------------------------------------------------------
# whole model: the packed forward (bongard/packing.py:228-318)
# --------------------------------------------------------------------------------------

def _positions(lengths):
    return torch.cat([torch.arange(n) for n in lengths]) if lengths else torch.zeros(0, dtype=torch.long)


def _layer(x, w, prefix, shape, index, lengths, positions, *, decoder, cross=None, owners=None,
           state_lengths=None, mlp=geglu_mlp, lin=linear):
    """One sandwich-norm layer (HF:477-503 encoder, HF:530-562 decoder)."""
    p = f'{prefix}.layers.{index}.'
    window, theta = shape.layer_window(index), shape.layer_theta(index)
    n = rmsnorm(x, w[p + 'pre_self_attn_layernorm.weight'], shape.eps)
    q = lin(n, w[p + 'self_attn.q_proj.weight']).view(-1, shape.q_heads, shape.head_dim)
    k = lin(n, w[p + 'self_attn.k_proj.weight']).view(-1, shape.kv_heads, shape.head_dim)
    v = lin(n, w[p + 'self_attn.v_proj.weight']).view(-1, shape.kv_heads, shape.head_dim)
    cos, sin = rope_tables(positions, shape.head_dim, theta, x.dtype)
    q, k = qk_norm_rope(q, k, w[p + 'self_attn.q_norm.weight'], w[p + 'self_attn.k_norm.weight'], cos, sin, shape.eps)
    if decoder:
        attn, _ = varlen_attention(q, k, v, lengths, shape.scale, window, cross=cross, owners=owners,
                                   state_lengths=state_lengths)
    else:
        attn, _ = varlen_attention(q, k, v, lengths, shape.scale, window)
    attn = lin(attn.reshape(-1, shape.q_dim), w[p + 'self_attn.o_proj.weight'])
    x = x + rmsnorm(attn, w[p + 'post_self_attn_layernorm.weight'], shape.eps)
    n = rmsnorm(x, w[p + 'pre_feedforward_layernorm.weight'], shape.eps)
    m = mlp(n, w[p + 'mlp.gate_proj.weight'], w[p + 'mlp.up_proj.weight'], w[p + 'mlp.down_proj.weight'])
    return x + rmsnorm(m, w[p + 'post_feedforward_layernorm.weight'], shape.eps)


def encode_packed(w, shape, states, *, mlp=geglu_mlp, lin=linear):
    """Encoder over a pack of states (bongard/packing.py:239-262; HF:794-854).  Returns [T,H]."""
    lengths = [len(s) for s in states]
    ids = torch.tensor([t for s in states for t in s], dtype=torch.long)
    table = w['encoder.text_model.embed_tokens.weight']
    x = embed(ids, table, w['encoder.text_model.embed_tokens.eoi_embedding'], shape.hidden, shape.eoi_token)
    positions = _positions(lengths)
    for index in range(shape.layers):
        x = _layer(x, w, 'encoder.text_model', shape, index, lengths, positions, decoder=False, mlp=mlp, lin=lin)
    return rmsnorm(x, w['encoder.text_model.norm.weight'], shape.eps)


def state_kv(w, shape, state, *, lin=linear):
    """bongard/model.py:135-139, 342-359: per decoder layer K = k_norm(k_proj(state)) with no
    rotation, V = v_proj(state).  Returns a list of (K, V) [S,Hkv,D]."""
    out = []
    for index in range(shape.layers):
        p = f'decoder.layers.{index}.self_attn.'
        k = lin(state, w[p + 'k_proj.weight']).view(-1, shape.kv_heads, shape.head_dim)
        v = lin(state, w[p + 'v_proj.weight']).view(-1, shape.kv_heads, shape.head_dim)
        out.append((rmsnorm(k, w[p + 'k_norm.weight'], shape.eps), v))
    return out


def decode_packed(w, shape, questions, owners, state_lengths, cross, *, mlp=geglu_mlp, lin=linear):
    """Decoder over one pack of questions (bongard/packing.py:273-306; HF:994-1087)."""
    lengths = [len(q) for q in questions]
    ids = torch.tensor([t for q in questions for t in q], dtype=torch.long)
    table = w['encoder.text_model.embed_tokens.weight']      # tied (HF:1100-1103)
    x = embed(ids, table, w['encoder.text_model.embed_tokens.eoi_embedding'], shape.hidden, shape.eoi_token)
    positions = _positions(lengths)
    for index in range(shape.layers):
        x = _layer(x, w, 'decoder', shape, index, lengths, positions, decoder=True, cross=cross[index],
                   owners=owners, state_lengths=state_lengths, mlp=mlp, lin=lin)
    return rmsnorm(x, w['decoder.norm.weight'], shape.eps)


def forward_packed(w, shape, requests, branch_batch_size=8, *, dtype=torch.float32, mlp=geglu_mlp, lin=linear):
    """bongard/packing.py:228-318 for distinct states: one encoder pass over all states, the
    state K/V projected once per decoder layer, questions decoded in groups of
    branch_batch_size in request order, candidate and decision rows read out and scored
    (bongard/model.py:520-529).  Returns [{qid: {'logits': [K], 'readouts': [K+1,H]}}]."""
    w = {k: v.to(dtype) for k, v in w.items()}
    states = [r.state for r in requests]
    state_lengths = [len(s) for s in states]
    state = encode_packed(w, shape, states, mlp=mlp, lin=lin)
    cross = state_kv(w, shape, state, lin=lin)
    members = [((i, qid), q) for i, r in enumerate(requests) for qid, q in r.questions.items()]
    readouts = {}
    for start in range(0, len(members), branch_batch_size):
        group = members[start:start + branch_batch_size]
        hidden = decode_packed(w, shape, [q.tokens for _, q in group], [key[0] for key, _ in group],
                               state_lengths, cross, mlp=mlp, lin=lin)
        offset = 0
        for key, q in group:
            rows = [offset + p for p in q.candidate_positions] + [offset + q.decision_position]
            readouts[key] = hidden[rows]
            offset += len(q.tokens)
    out = [dict() for _ in requests]
    for key, q in members:
        r = readouts[key]
        h, g = r[:-1], r[-1:].expand(len(r) - 1, -1)
        logits = judgment_head(h, g, w['head.w.weight'], w['head.candidate.weight'], w['head.global_readout.weight'])
        out[key[0]][key[1]] = {'logits': logits, 'readouts': r}
    return out
