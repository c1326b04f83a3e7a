"""Hugging Face T5Gemma2 backbones for the drop-in path.

`build_backbone` creates the `transformers` T5Gemma2Model of a ModelShape and loads
Hugging Face-named weights into it; `PackedJudge` drives the (module-substituted) backbone
through the same sequence of calls as the reference's packed forward
(bongard/packing.py:228-318): one encoder call over the packed states with `packed_layout=`,
the state K/V of every decoder layer, decoder layers called with `question_layout=` and
`packed_cross=`, readout rows, judgment head.  It exists so that the substituted modules can
be exercised - and checked against the reference's fixtures - on a host that has
`transformers` but not the reference package.
"""

from __future__ import annotations

import torch

from . import ops
from .packing import packed_layout
from .workload import ModelShape


def hf_config(shape: ModelShape, max_positions=131072):
    from transformers import T5Gemma2Config

    text = dict(
        vocab_size=shape.vocab, hidden_size=shape.hidden, intermediate_size=shape.intermediate,
        num_hidden_layers=shape.layers, num_attention_heads=shape.q_heads, num_key_value_heads=shape.kv_heads,
        head_dim=shape.head_dim, query_pre_attn_scalar=shape.query_pre_attn_scalar, sliding_window=shape.window,
        layer_types=list(shape.layer_types), max_position_embeddings=max_positions,
        rope_parameters={'sliding_attention': {'rope_type': 'default', 'rope_theta': shape.theta_local},
                         'full_attention': {'rope_type': 'default', 'rope_theta': shape.theta_global}})
    vision = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                  image_size=28, patch_size=14)
    return T5Gemma2Config(encoder=dict(text_config=text, vision_config=vision, mm_tokens_per_image=4),
                          decoder=dict(text))


def build_backbone(shape: ModelShape, weights, device='cuda', dtype=torch.bfloat16):
    from transformers import T5Gemma2Model

    backbone = T5Gemma2Model(hf_config(shape)).eval()
    state = {k: v for k, v in weights.items() if not k.startswith('head.')}
    for key in ('weight', 'eoi_embedding'):
        state[f'decoder.embed_tokens.{key}'] = state[f'encoder.text_model.embed_tokens.{key}']
    missing, unexpected = backbone.load_state_dict(state, strict=False)
    if unexpected or any('vision' not in m and 'multi_modal' not in m for m in missing):
        raise ValueError(f'weights do not match the backbone: missing {missing}, unexpected {unexpected}')
    return backbone.to(device=device, dtype=dtype)


class PackedJudge:
    """Packed forward over a Hugging Face backbone whose hot-path modules were substituted."""

    def __init__(self, backbone, head, eoi_token=256_000):
        self.backbone = backbone
        self.device = next(backbone.parameters()).device
        self.head = {k: head[k].to(self.device, torch.bfloat16).contiguous()
                     for k in ('head.w.weight', 'head.candidate.weight', 'head.global_readout.weight')}

    def ids(self, values):
        return torch.tensor([values], dtype=torch.long, device=self.device)

    @torch.inference_mode()
    def encode(self, states):
        layout = packed_layout([len(s) for s in states], [], self.device)
        empty = torch.empty(0, device=self.device)
        out = self.backbone.encoder(
            input_ids=self.ids([t for s in states for t in s]), position_ids=layout.positions,
            attention_mask={'full_attention': empty, 'sliding_attention': empty}, packed_layout=layout, use_cache=False)
        return out.last_hidden_state

    @torch.inference_mode()
    def state_kv(self, state):
        """Per decoder layer (keys, values) [1, Hkv, S, D] (bongard/model.py:342-359)."""
        return [layer.self_attn._cross(None, state, None) for layer in self.backbone.decoder.layers]

    @torch.inference_mode()
    def decode(self, questions, owners, state_lengths, state, cross):
        decoder = self.backbone.decoder
        layout = packed_layout([len(q) for q in questions], [], self.device, owners=owners, state_lengths=state_lengths)
        hidden = decoder.embed_tokens(self.ids([t for q in questions for t in q]))
        embeddings = {t: decoder.rotary_emb(hidden, layout.positions, t) for t in set(decoder.config.layer_types)}
        empty = torch.empty(0, device=self.device)
        for index, layer in enumerate(decoder.layers):
            hidden = layer(hidden, embeddings[decoder.config.layer_types[index]], empty, layout.positions, None, False,
                           state, question_layout=layout, packed_cross=cross[index])
        return decoder.norm(hidden)[0]

    @torch.inference_mode()
    def forward_packed(self, requests, branch_batch_size=8):
        state = self.encode([r.state for r in requests])
        cross = self.state_kv(state)
        state_lengths = [len(r.state) for r in requests]
        members = [((i, qid), q) for i, r in enumerate(requests) for qid, q in r.questions.items()]
        out = [dict() for _ in requests]
        for start in range(0, len(members), branch_batch_size):
            group = members[start:start + branch_batch_size]
            hidden = self.decode([q.tokens for _, q in group], [key[0] for key, _ in group], state_lengths, state, cross)
            offset = 0
            for key, q in group:
                cand = [offset + p for p in q.candidate_positions]
                rows = torch.tensor([cand, [offset + q.decision_position] * len(cand)], dtype=torch.int32, device=self.device)
                logits = ops.judgment_head(hidden, rows[0], rows[1], self.head['head.w.weight'],
                                           self.head['head.candidate.weight'], self.head['head.global_readout.weight'])
                readouts = hidden.index_select(0, torch.tensor(cand + [offset + q.decision_position], device=self.device))
                out[key[0]][key[1]] = {'logits': logits, 'readouts': readouts}
                offset += len(q.tokens)
        ops.read_status()
        return out
