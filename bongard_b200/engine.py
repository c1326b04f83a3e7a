"""Packed inference engine: the reference's forward_packed (bongard/packing.py:228-318) as a
straight chain of C-ABI kernels over Hugging Face-named weights.

Per layer (sandwich norms, transformers modeling_t5gemma2.py:477-503 / 530-562):

    qkv  = linear(n, [Wq; Wk; Wv])            one stacked GEMM (bongard/te_linear.py:47-55)
    q, k = qk_norm_rope(qkv)                  in place, v stays a view of the same buffer
    a    = varlen_attention(q, k, v [, state K/V])
    o    = linear(a, Wo)
    x   += post_norm(o);  n2 = pre_ffn_norm(x)                 one fused kernel
    h    = gelu_tanh(n2 Wg^T) * (n2 Wu^T)                      one GEMM with the GeGLU epilogue
    d    = linear(h, Wd)
    x   += post_norm(d);  n  = next layer's pre_attn_norm(x)   one fused kernel

States are encoded in packs of at most `encoder_pack_tokens`; for each pack the decoder's
state K/V of every layer are projected once (bongard/model.py:342-359) and all questions of
the pack's requests are decoded in packs of whole 8-question groups.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from . import ops
from .workload import ModelShape, embed_scale

BF16 = torch.bfloat16


@dataclass
class LayerWeights:
    wqkv: object             # bf16 tensors, ops.Fp8Weight under linears='fp8', ops.Mxfp8Tensor under 'mxfp8'
    wkv: object              # the k|v rows of wqkv (decoder: projects the shared state)
    wo: object
    wgu: object
    wdown: object
    pre_attn: torch.Tensor
    post_attn: torch.Tensor
    pre_ffn: torch.Tensor
    post_ffn: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor


def _stack_layer(w, prefix, device, linears='bf16', state_kv=False):
    g = lambda name: w[prefix + name].to(device=device, dtype=BF16)   # noqa: E731
    fp8 = linears != 'bf16'
    conv = {'bf16': lambda t: t, 'fp8': ops.quantize_weight, 'mxfp8': ops.quantize_mxfp8}[linears]
    wqkv = torch.cat([g('self_attn.q_proj.weight'), g('self_attn.k_proj.weight'), g('self_attn.v_proj.weight')]).contiguous()
    q_rows = w[prefix + 'self_attn.q_proj.weight'].shape[0]
    return LayerWeights(
        wqkv=conv(wqkv),
        wkv=(conv(wqkv[q_rows:].contiguous()) if fp8 else wqkv[q_rows:]) if state_kv else None,
        wo=conv(g('self_attn.o_proj.weight').contiguous()),
        wgu=conv(torch.cat([g('mlp.gate_proj.weight'), g('mlp.up_proj.weight')]).contiguous()),
        wdown=conv(g('mlp.down_proj.weight').contiguous()),
        pre_attn=g('pre_self_attn_layernorm.weight'), post_attn=g('post_self_attn_layernorm.weight'),
        pre_ffn=g('pre_feedforward_layernorm.weight'), post_ffn=g('post_feedforward_layernorm.weight'),
        q_norm=g('self_attn.q_norm.weight'), k_norm=g('self_attn.k_norm.weight'))


class JudgmentEngine:
    """A full replica of the judgment model on one GPU."""

    def __init__(self, weights, shape: ModelShape, device='cuda', *, encoder_pack_tokens=65536,
                 decoder_pack_tokens=32768, linears='bf16', residual=None, wide_outputs=True):
        ops.device_check()
        if linears not in ('bf16', 'fp8', 'mxfp8'):
            raise ValueError("linears must be 'bf16', 'fp8' or 'mxfp8'")
        supports_fp32 = linears != 'mxfp8' and shape.hidden % 256 == 0 and shape.hidden <= 3072
        if residual is None:
            residual = 'fp32' if supports_fp32 else 'bf16'
        if residual not in ('bf16', 'fp32'):
            raise ValueError("residual must be 'bf16' or 'fp32'")
        if residual == 'fp32' and not supports_fp32:
            raise ValueError('the fp32 residual stream needs a hidden size that is a multiple of 256 (up to 3072) and '
                             'bf16 or fp8 linears')
        # Precision of what flows between the layers.
        # 'fp32' (default where supported): the residual stream stays fp32 (embedding, residual adds, the input of every
        #   pre-norm) and, with wide_outputs (default), the output and down projections hand their fp32 accumulators to
        #   the post-norm unrounded.  GEMM and attention operands are bf16 as before.  This is the arithmetic of the
        #   reference run in float32 up to the rounding of the tensor-core operands; it brings the probabilities of
        #   the tiny model within 1e-3 of the reference's fp32 result (0.8e-3) for 3 % of the throughput.
        # 'bf16': the stream and the post-norm results are rounded to bf16 exactly where the reference's bf16 module
        #   chain rounds them (1.7e-3 on the same case, the reference's own bf16 path: 1.8e-3).
        self.residual = residual
        # with the fp32 stream: also hand the post-norms the output and down projections unrounded (fp32)
        self.fp32_projection_outputs = bool(wide_outputs) and residual == 'fp32'
        self.linears, fp8 = linears, linears
        self.shape, self.device = shape, torch.device(device)
        self.encoder_pack_tokens, self.decoder_pack_tokens = encoder_pack_tokens, decoder_pack_tokens
        g = lambda name: weights[name].to(device=self.device, dtype=BF16).contiguous()   # noqa: E731
        self.table = g('encoder.text_model.embed_tokens.weight')
        self.eoi = g('encoder.text_model.embed_tokens.eoi_embedding')
        self.enc_norm, self.dec_norm = g('encoder.text_model.norm.weight'), g('decoder.norm.weight')
        self.enc = [_stack_layer(weights, f'encoder.text_model.layers.{i}.', self.device, fp8) for i in range(shape.layers)]
        self.dec = [_stack_layer(weights, f'decoder.layers.{i}.', self.device, fp8, True) for i in range(shape.layers)]
        self.head_w, self.head_c, self.head_g = g('head.w.weight'), g('head.candidate.weight'), g('head.global_readout.weight')
        # per stack, as a checkpoint may override either (bongard/model.py:632-637)
        self.embed_scale_enc = self.embed_scale_dec = embed_scale(shape, BF16 if residual == 'bf16' else torch.float32)
        self.launches = 0          # kernels launched by this library (for reporting)
        # The serving path lets stacks of up to 256 tokens use the split-K weight-streaming GEMM.  The
        # packed engine keeps it off, so that where a pack boundary falls never changes a result bit.
        self.few_rows_kernels = False
        self.programmatic_launch = False   # set by the serving path (serving.Predictor)
        # Opt-in: apply QK-norm + RoPE inside the q|k|v GEMM epilogue (bg_gemm_bf16_qkv_rope).  Alone the
        # fused projection is 6 % faster than projection + separate kernel, but inside the power-capped
        # step the extra epilogue arithmetic slows the GEMM by as much as the separate pass cost.
        self.fuse_qkv_rope = False

    # ------------------------------------------------------------------ host-side preparation
    def _window_key(self, index, longest, decoder):
        """A window that covers every segment of the pack is the same as no window
        (the reference uses the same test to route layers to its dense kernel,
        bongard/packing.py:84-85)."""
        window = self.shape.layer_window(index)
        if window is None:
            return None
        reach = window if decoder else (window + 1) // 2
        return None if longest <= reach else window

    def _host_pack(self, sequences, *, owners=None, state_lengths=None, readout=None):
        s = self.shape
        lengths = [len(seq) for seq in sequences]
        total = sum(lengths)
        ids = np.empty(total, dtype=np.int64)
        positions = np.empty(total, dtype=np.int32)
        offset = 0
        for seq, n in zip(sequences, lengths):
            ids[offset:offset + n] = seq
            positions[offset:offset + n] = np.arange(n, dtype=np.int32)
            offset += n
        decoder = owners is not None
        longest = max(lengths)
        keys = [self._window_key(i, longest, decoder) for i in range(s.layers)]
        plans, parts, cursor = {}, [positions], total
        for key in dict.fromkeys(keys):
            hp = ops.make_host_plan(lengths, key, group=s.q_heads // s.kv_heads, owners=owners, state_lengths=state_lengths,
                                    head_dim=s.head_dim)
            plans[key] = (cursor, hp)
            parts.append(hp.packed)
            cursor += hp.packed.size
        rows = None
        if readout is not None:
            rows = (cursor, len(readout[0]))
            parts.append(np.asarray(readout[0] + readout[1], dtype=np.int32))
        pairs = sum(plans[k][1].pairs for k in keys)
        return HostPack(torch.from_numpy(ids).pin_memory(), torch.from_numpy(np.concatenate(parts)).pin_memory(),
                        total, keys, plans, rows, pairs, longest)

    def prepare(self, requests, branch_batch_size=8, state_owners=None):
        """Host-side layout of a batch: token ids, positions, attention plans and readout rows
        of every encoder and decoder pack, in pinned buffers ready for one copy each.

        Requests of one pack that share an owner and a state (`state_owners`, as in the reference's
        forward_packed, bongard/packing.py:229-238) are encoded once and share the state K/V."""
        batch = HostBatch()
        s = self.shape
        owners = list(range(len(requests))) if state_owners is None else list(state_owners)
        if len(owners) != len(requests):
            raise ValueError('state_owners must match requests')
        for pack in self._request_packs(requests):
            reqs = [requests[i] for i in pack]
            states, rows, row_of = [], {}, []
            for i, r in zip(pack, reqs):
                key = (owners[i], r.state_key)
                if key not in rows:
                    rows[key] = len(states)
                    states.append(r.state)
                row_of.append(rows[key])
            state_lengths = [len(st) for st in states]
            enc = self._host_pack(states)
            members = [((row_of[local], qid), q) for local, r in enumerate(reqs) for qid, q in r.questions.items()]
            decs = []
            for qpack in self._question_packs(members, branch_batch_size):
                cand, dec, offset = [], [], 0
                for _, q in qpack:
                    cand.extend(offset + p for p in q.candidate_positions)
                    dec.extend([offset + q.decision_position] * len(q.candidate_positions))
                    batch.sizes.append(len(q.candidate_positions))
                    offset += len(q.tokens)
                decs.append(self._host_pack([q.tokens for _, q in qpack], owners=[key[0] for key, _ in qpack],
                                            state_lengths=state_lengths, readout=(cand, dec)))
            batch.packs.append((enc, decs))
            tokens = enc.tokens + sum(d.tokens for d in decs)
            batch.gemm_flops += 2 * s.params_per_layer * s.layers * tokens + 2 * s.layers * enc.tokens * s.hidden * 2 * s.kv_dim
            batch.attn_flops += 4 * s.head_dim * s.q_heads * (enc.pairs + sum(d.pairs for d in decs))
            batch.h2d_bytes += sum(p.ids.numel() * 8 + p.ints.numel() * 4 for p in [enc] + decs)
        batch.offsets = torch.tensor([0] + batch.sizes, dtype=torch.int64).cumsum(0).to(torch.int32).pin_memory()
        batch.h2d_bytes += batch.offsets.numel() * 4
        return batch

    def stage(self, batch):
        """Copy a prepared batch to the device (two async copies per pack)."""
        staged = []
        for enc, decs in batch.packs:
            staged.append((enc.to(self.device), [d.to(self.device) for d in decs]))
        return staged, batch.offsets.to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ device execution
    def _freqs(self, index):
        return ops.inv_freq(self.shape.head_dim, self.shape.layer_theta(index), self.device)

    def _lin(self, x, w, geglu=False):
        if isinstance(w, ops.Fp8Weight):
            return ops.linear_fp8(x, w, geglu=geglu)
        if isinstance(w, ops.Mxfp8Tensor):
            return ops.linear_mxfp8(x, w, geglu=geglu)
        few = self.few_rows_kernels
        return ops.linear_geglu(x, w, few_rows=few) if geglu else ops.linear(x, w, few_rows=few)

    def _stack(self, layers, final_norm, pack, cross=None):
        s = self.shape
        scale = self.embed_scale_enc if layers is self.enc else self.embed_scale_dec
        x = ops.embed(pack.ids, self.table, self.eoi, scale, s.eoi_token,
                      dtype=BF16 if self.residual == 'bf16' else torch.float32)
        mx = self.linears == 'mxfp8'          # norms hand the GEMMs MXFP8 directly: no bf16 copy of a normed row
        n = ops.rmsnorm_mxfp8(x, layers[0].pre_attn, s.eps) if mx else ops.rmsnorm(x, layers[0].pre_attn, s.eps)
        t = x.shape[0]
        qd, kd = s.q_dim, s.kv_dim
        self.launches += 2
        for index, lw in enumerate(layers):
            fused = (self.fuse_qkv_rope and pack.longest > 0 and not self.few_rows_kernels
                     and isinstance(lw.wqkv, torch.Tensor))
            if fused:
                # QK-norm + RoPE ride in the projection's epilogue: one pass less over q and k
                table = ops.rope_table(s.head_dim, s.layer_theta(index), pack.longest, self.device)
                qkv = ops.linear_qkv_rope(n, lw.wqkv, qd, kd, s.head_dim, lw.q_norm, lw.k_norm, pack.positions, table, s.eps)
            else:
                qkv = self._lin(n, lw.wqkv)
            q = qkv[:, :qd].view(t, s.q_heads, s.head_dim)
            k = qkv[:, qd:qd + kd].view(t, s.kv_heads, s.head_dim)
            v = qkv[:, qd + kd:].view(t, s.kv_heads, s.head_dim)
            if not fused:
                # with the positions' bound known, the angles come from a per-(theta) table of the same values
                table = (ops.rope_table(s.head_dim, s.layer_theta(index), pack.longest, self.device)
                         if pack.longest > 0 else None)
                ops.qk_norm_rope_(q, k, lw.q_norm, lw.k_norm, pack.positions, self._freqs(index), s.eps, table=table)
            a = ops.varlen_attention(q, k, v, pack.plans[pack.keys[index]], s.scale,
                                     None if cross is None else cross[index])
            # (not on the latency path, whose few-row weight-streaming GEMM writes bf16)
            wide = self.fp32_projection_outputs and not self.few_rows_kernels and isinstance(lw.wo, torch.Tensor)
            o = ops.linear_f32out(a, lw.wo) if wide else self._lin(a, lw.wo)
            n2 = (ops.add_rmsnorm_mxfp8_ if mx else ops.add_rmsnorm_)(o, lw.post_attn, x, lw.pre_ffn, s.eps)
            if isinstance(lw.wgu, ops.Mxfp8Tensor):
                d = ops.mlp_mxfp8(n2, lw.wgu, lw.wdown)        # the hidden activation stays MXFP8
            else:
                h = self._lin(n2, lw.wgu, geglu=True)
                d = ops.linear_f32out(h, lw.wdown) if wide else self._lin(h, lw.wdown)
            last = index + 1 == len(layers)
            nxt = final_norm if last else layers[index + 1].pre_attn
            n = (ops.add_rmsnorm_mxfp8_ if mx and not last else ops.add_rmsnorm_)(d, lw.post_ffn, x, nxt, s.eps)
            self.launches += 7 if fused else 8
        return n

    def state_kv(self, state):
        """Per decoder layer (K, V) [S, kv_heads, D]: K = k_norm(k_proj(state)) without rotation,
        V = v_proj(state) (bongard/model.py:135-139)."""
        s = self.shape
        out = []
        if self.linears == 'mxfp8':
            state = ops.quantize_mxfp8(state)          # one quantisation serves every layer's projection
        for lw in self.dec:
            kv = self._lin(state, lw.wkv)
            k = kv[:, :s.kv_dim].view(-1, s.kv_heads, s.head_dim)
            v = kv[:, s.kv_dim:].view(-1, s.kv_heads, s.head_dim)
            ops.qk_norm_rope_(None, k, None, lw.k_norm, None, None, s.eps, rotate=False)
            out.append((k, v))
            self.launches += 2
        return out

    def execute(self, staged, *, keep_hidden=False):
        """Run a staged batch; returns candidate logits fp32 [n_candidates] (device)."""
        from . import _lib
        lib = _lib.load()
        lib.bg_set_programmatic_launch(1 if self.programmatic_launch else 0)
        try:
            return self._execute(staged, keep_hidden)
        finally:
            lib.bg_set_programmatic_launch(0)

    def _execute(self, staged, keep_hidden):
        logits, hidden_rows = [], []
        for enc, decs in staged:
            state = self._stack(self.enc, self.enc_norm, enc)
            cross = self.state_kv(state)
            for dec in decs:
                hidden = self._stack(self.dec, self.dec_norm, dec, cross)
                logits.append(ops.judgment_head(hidden, dec.cand_rows, dec.dec_rows, self.head_w, self.head_c, self.head_g))
                self.launches += 1
                if keep_hidden:
                    hidden_rows.append((hidden, dec.cand_rows, dec.dec_rows))
            del cross, state
        out = torch.cat(logits) if logits else torch.zeros(0, device=self.device)
        return (out, hidden_rows) if keep_hidden else out

    def probabilities(self, logits, offsets, temperature=1.0):
        self.launches += 1
        return ops.candidate_softmax(logits, offsets, temperature)

    # ------------------------------------------------------------------ whole requests
    def _request_packs(self, requests):
        packs, current, tokens = [], [], 0
        for index, r in enumerate(requests):
            n = len(r.state)
            if current and tokens + n > self.encoder_pack_tokens:
                packs.append(current)
                current, tokens = [], 0
            current.append(index)
            tokens += n
        if current:
            packs.append(current)
        return packs

    def _question_packs(self, members, branch_batch_size):
        """Whole groups of branch_batch_size questions (request order) up to decoder_pack_tokens."""
        groups = [members[i:i + branch_batch_size] for i in range(0, len(members), branch_batch_size)]
        packs, current, tokens = [], [], 0
        for group in groups:
            n = sum(len(q.tokens) for _, q in group)
            if current and tokens + n > self.decoder_pack_tokens:
                packs.append(current)
                current, tokens = [], 0
            current.extend(group)
            tokens += n
        if current:
            packs.append(current)
        return packs

    @staticmethod
    def _split(flat, sizes, requests):
        out, cursor, it = [], 0, iter(sizes)
        for r in requests:
            answers = {}
            for qid in r.questions:
                n = next(it)
                answers[qid] = flat[cursor:cursor + n]
                cursor += n
            out.append(answers)
        return out

    @torch.inference_mode()
    def judge(self, requests, branch_batch_size=8, temperature=1.0):
        """Per-candidate probabilities of every question: host token ids in, ONE device-to-host
        copy of float64 probabilities out (bongard/inference.py:305-321 reads logits back once
        per request and runs `probabilities` on the host; here the softmax runs on the device)."""
        batch = self.prepare(requests, branch_batch_size)
        staged, offsets = self.stage(batch)
        probs = self.probabilities(self.execute(staged), offsets, temperature)
        host = probs.cpu()
        ops.read_status()
        return self._split(host, batch.sizes, requests)

    @torch.inference_mode()
    def forward_packed(self, requests, branch_batch_size=8, state_owners=None):
        """Same result structure as the reference's forward_packed: one dict per request,
        {qid: {'logits': [K], 'readouts': [K+1, hidden]}} (bongard/packing.py:316-318)."""
        batch = self.prepare(requests, branch_batch_size, state_owners)
        staged, _ = self.stage(batch)
        logits, hidden_rows = self.execute(staged, keep_hidden=True)
        readouts = []
        for hidden, cand, dec in hidden_rows:
            cand, dec = cand.tolist(), dec.tolist()
            i = 0
            while i < len(cand):
                j = i
                while j < len(cand) and dec[j] == dec[i]:
                    j += 1
                readouts.append(hidden.index_select(0, torch.tensor(cand[i:j] + [dec[i]], device=self.device)))
                i = j
        out = self._split(logits, batch.sizes, requests)
        k = 0
        for answers in out:
            for qid in answers:
                answers[qid] = {'logits': answers[qid], 'readouts': readouts[k]}
                k += 1
        ops.read_status()
        return out


@dataclass
class DevicePack:
    ids: torch.Tensor
    positions: torch.Tensor
    keys: list
    plans: dict
    cand_rows: torch.Tensor = None
    dec_rows: torch.Tensor = None
    longest: int = 0         # longest segment = positions in use (0: unknown, the fused RoPE epilogue is skipped)


@dataclass
class HostPack:
    ids: torch.Tensor        # pinned int64 [T]
    ints: torch.Tensor       # pinned int32 [positions | plans... | readout rows]
    tokens: int
    keys: list               # per layer: the window its attention plan was built for
    plans: dict              # window -> (offset into ints, ops.HostPlan)
    rows: tuple              # (offset, n_candidates) or None
    pairs: int               # visible attention pairs summed over layers
    longest: int = 0         # longest segment of the pack

    def to(self, device):
        ids = self.ids.to(device, non_blocking=True)
        ints = self.ints.to(device, non_blocking=True)
        plans = {k: hp.view(ints[o:o + hp.packed.size]) for k, (o, hp) in self.plans.items()}
        pack = DevicePack(ids, ints[:self.tokens], self.keys, plans, longest=self.longest)
        if self.rows is not None:
            o, n = self.rows
            pack.cand_rows, pack.dec_rows = ints[o:o + n], ints[o + n:o + 2 * n]
        return pack


@dataclass
class HostBatch:
    packs: list = field(default_factory=list)
    sizes: list = field(default_factory=list)     # candidates per question, request/question order
    offsets: torch.Tensor = None
    gemm_flops: int = 0
    attn_flops: int = 0
    h2d_bytes: int = 0
