"""Generate tests/golden/*.npz by running the reference itself on CPU.

Run with a checkout of the reference on the import path ($BONGARD_REFERENCE names its directory):

    python tests/golden/make_golden.py

It imports the reference's own modules (bongard.model.JudgmentModel, bongard.packing,
bongard.attention, bongard.inference) and the Hugging Face T5Gemma2 model they wrap,
feeds them the seeded weights and requests of bongard_b200.workload, and stores inputs
and outputs.  The fixtures are what travels: tests replay them without the reference.
"""

import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, os.environ.get('BONGARD_REFERENCE', str(ROOT.parent / 'reference')))

from bongard_b200 import workload as wl  # noqa: E402

from bongard import attention as ref_attention  # noqa: E402
from bongard import packing as ref_packing  # noqa: E402
from bongard.compiler import Question as RefQuestion, Request as RefRequest  # noqa: E402
from bongard.inference import probabilities as ref_probabilities  # noqa: E402
from bongard.model import JudgmentHead, JudgmentModel  # noqa: E402
from transformers import T5Gemma2Config, T5Gemma2Model  # noqa: E402
from transformers.models.t5gemma2.modeling_t5gemma2 import (  # noqa: E402
    T5Gemma2MLP, T5Gemma2RMSNorm, T5Gemma2RotaryEmbedding, T5Gemma2TextScaledWordEmbedding)

OUT = Path(__file__).resolve().parent


def hf_config(shape: wl.ModelShape):
    text = dict(
        vocab_size=shape.vocab, hidden_size=shape.hidden, intermediate_size=shape.intermediate,
        num_hidden_layers=shape.layers, num_attention_heads=shape.q_heads,
        num_key_value_heads=shape.kv_heads, head_dim=shape.head_dim,
        query_pre_attn_scalar=shape.query_pre_attn_scalar, sliding_window=shape.window,
        layer_types=list(shape.layer_types), max_position_embeddings=8192,
        rope_parameters={'sliding_attention': {'rope_type': 'default', 'rope_theta': shape.theta_local},
                         'full_attention': {'rope_type': 'default', 'rope_theta': shape.theta_global}})
    vision = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                  image_size=28, patch_size=14)
    return T5Gemma2Config(encoder=dict(text_config=text, vision_config=vision, mm_tokens_per_image=4),
                          decoder=dict(text))


def reference_model(shape, weights, dtype):
    compiler = types.SimpleNamespace(tokenizer=types.SimpleNamespace(pad_token_id=0), eos=1)
    model = JudgmentModel(T5Gemma2Model(hf_config(shape)), compiler, dtype=dtype).eval()
    state = {}
    for name, value in weights.items():
        if name.startswith('head.'):
            state[name] = value
        else:
            state['backbone.' + name] = value
            if name.startswith('encoder.text_model.embed_tokens.'):
                state['backbone.decoder.embed_tokens.' + name.rsplit('.', 1)[1]] = value
    missing, unexpected = model.load_state_dict({k: v.to(dtype) for k, v in state.items()}, strict=False)
    assert not unexpected, unexpected
    assert all('vision' in m or 'multi_modal' in m for m in missing), missing
    return model


def to_ref(requests):
    return [RefRequest(r.state, {qid: RefQuestion(q.keys, q.tokens, q.candidate_positions, q.decision_position,
                                                  q.instruction_tokens) for qid, q in r.questions.items()},
                       r.input_tokens) for r in requests]


def flat_logits(result):
    return np.concatenate([v['logits'].float().numpy() for answers in result for v in answers.values()])


def flat_probs(result):
    return np.concatenate([ref_probabilities(v['logits'].float(), 1.0).numpy()
                           for answers in result for v in answers.values()])


@torch.inference_mode()
def end_to_end(name, shape, seed, norm_std, requests):
    weights = wl.make_weights(shape, seed, norm_std=norm_std)
    ref_requests = to_ref(requests)
    out = {}
    for dtype, tag in ((torch.float32, 'fp32'), (torch.bfloat16, 'bf16')):
        model = reference_model(shape, weights, dtype)
        serving = [model(r) for r in ref_requests]
        model.packing, model.packing_attention = True, 'triton'
        packed = model(ref_requests)
        out[f'logits_serving_{tag}'] = flat_logits(serving)
        out[f'logits_packed_{tag}'] = flat_logits(packed)
        out[f'probs_serving_{tag}'] = flat_probs(serving)
        out[f'probs_packed_{tag}'] = flat_probs(packed)
        if tag == 'fp32':
            out['readouts_packed_fp32'] = np.concatenate(
                [v['readouts'].float().numpy() for answers in packed for v in answers.values()])
    out['weights_checksum'] = np.array([float(sum(v.double().abs().sum() for v in weights.values()))])
    np.savez_compressed(OUT / f'{name}.npz', **out)
    print(name, 'serving vs packed fp32', np.abs(out['logits_serving_fp32'] - out['logits_packed_fp32']).max(),
          'fp32 vs bf16 probs', np.abs(out['probs_packed_fp32'] - out['probs_packed_bf16']).max(),
          'bf16 serving vs packed probs', np.abs(out['probs_serving_bf16'] - out['probs_packed_bf16']).max())


@torch.inference_mode()
def op_level():
    rng = np.random.Generator(np.random.PCG64(7))

    def randn(*dims, std=1.0):
        return torch.from_numpy(rng.standard_normal(dims, dtype=np.float32) * np.float32(std))

    out = {}
    # RMSNorm, fp32 and bf16
    x, w = randn(7, 256), randn(256, std=0.2)
    norm = T5Gemma2RMSNorm(256, eps=1e-6)
    norm.weight.data.copy_(w)
    out.update(norm_x=x.numpy(), norm_w=w.numpy(), norm_y=norm(x).numpy(),
               norm_y_bf16=norm(x.bfloat16()).float().numpy())

    # scaled embedding with the end-of-image override
    table, eoi = randn(300, 64, std=0.02), randn(64, std=0.1)
    emb = T5Gemma2TextScaledWordEmbedding(300, 64, 0, embed_scale=64 ** 0.5, eoi_token_index=123)
    emb.weight.data.copy_(table)
    emb.eoi_embedding.data.copy_(eoi)
    ids = torch.tensor([[5, 123, 299, 0, 123, 17]])
    out.update(emb_table=table.numpy(), emb_eoi=eoi.numpy(), emb_ids=ids[0].numpy(), emb_y=emb(ids)[0].numpy(),
               emb_y_bf16=emb.bfloat16()(ids)[0].float().numpy())

    # project_qk on a real HF attention module of the tiny shape (bongard/attention.py:172-180)
    shape = wl.TINY
    backbone = T5Gemma2Model(hf_config(shape)).eval()
    attn = backbone.encoder.text_model.layers[0].self_attn
    for p in attn.parameters():
        p.data.copy_(randn(*p.shape, std=0.2 if p.ndim == 1 else 0.05))
    lengths = [5, 17, 1, 33]
    positions = torch.cat([torch.arange(n) for n in lengths])[None]
    hidden = randn(1, sum(lengths), shape.hidden)
    rotary = T5Gemma2RotaryEmbedding(backbone.config.encoder.text_config)
    pe = rotary(hidden, positions, 'sliding_attention')
    q, k = ref_attention.project_qk(attn, hidden, pe, 'reference')
    out.update(qk_hidden=hidden[0].numpy(), qk_positions=positions[0].numpy(),
               qk_wq=attn.q_proj.weight.detach().numpy(), qk_wk=attn.k_proj.weight.detach().numpy(),
               qk_qnorm=attn.q_norm.weight.detach().numpy(), qk_knorm=attn.k_norm.weight.detach().numpy(),
               qk_q=q[0].transpose(0, 1).numpy(), qk_k=k[0].transpose(0, 1).numpy(),
               qk_cos=pe[0][0].numpy(), qk_sin=pe[1][0].numpy())
    # the decoder's shared state keys: k_norm, no rotation (bongard/model.py:135-139)
    from bongard.model import project_state_kv
    sk, sv = project_state_kv(attn, hidden)
    out.update(state_k=sk[0].transpose(0, 1).numpy(), state_v=sv[0].transpose(0, 1).numpy(),
               qk_wv=attn.v_proj.weight.detach().numpy())

    # packed attention through the reference's CPU dispatcher (dense masks + SDPA)
    hq, hkv, d = 4, 2, 64
    t = sum(lengths)
    q, k, v = randn(1, hq, t, d), randn(1, hkv, t, d), randn(1, hkv, t, d)
    out.update(att_q=q[0].transpose(0, 1).numpy(), att_k=k[0].transpose(0, 1).numpy(),
               att_v=v[0].transpose(0, 1).numpy(), att_lengths=np.array(lengths))
    cpu = torch.device('cpu')
    for window in (None, 4, 5, 16):
        layout = ref_packing.packed_layout(lengths, [window], cpu, backend='triton')
        o = ref_packing.layout_attention(q, k, v, layout, 0.125, window)
        out[f'att_enc_w{window}'] = o[0].transpose(0, 1).numpy()
    state_lengths, owners = [9, 40], [0, 0, 1, 1]
    ck, cv = randn(1, hkv, sum(state_lengths), d), randn(1, hkv, sum(state_lengths), d)
    out.update(att_ck=ck[0].transpose(0, 1).numpy(), att_cv=cv[0].transpose(0, 1).numpy(),
               att_state_lengths=np.array(state_lengths), att_owners=np.array(owners))
    for window in (None, 4, 16):
        layout = ref_packing.packed_layout(lengths, [window], cpu, owners=owners, state_lengths=state_lengths,
                                           backend='triton')
        o = ref_packing.layout_attention(q, k, v, layout, 0.125, window, (ck, cv))
        out[f'att_dec_w{window}'] = o[0].transpose(0, 1).numpy()
    # the serving path's two-partition form must agree (bongard/attention.py:122-169)
    q1, k1, v1 = q[:, :, 5:22], k[:, :, 5:22], v[:, :, 5:22]
    mask = (torch.arange(17)[:, None] - torch.arange(17)[None, :] >= 0)[None]
    own = ref_attention.partition_attention(q1, k1, v1, mask, shared=False, scale=0.125)
    shared = ref_attention.partition_attention(q1, ck[:, :, :9], cv[:, :, :9], shared=True, scale=0.125)
    out['att_partition_seg1'] = ref_attention.merge_partitions([own, shared])[0].transpose(0, 1).numpy()

    # gated MLP
    mlp = T5Gemma2MLP(backbone.config.encoder.text_config).eval()
    for p in mlp.parameters():
        p.data.copy_(randn(*p.shape, std=0.05))
    x = randn(9, shape.hidden)
    out.update(mlp_x=x.numpy(), mlp_gate=mlp.gate_proj.weight.detach().numpy(),
               mlp_up=mlp.up_proj.weight.detach().numpy(), mlp_down=mlp.down_proj.weight.detach().numpy(),
               mlp_y=mlp(x).numpy())

    # judgment head and probabilities
    head = JudgmentHead(256)
    for p in head.parameters():
        p.data.copy_(randn(*p.shape, std=0.05))
    h, g = randn(6, 256), randn(1, 256).expand(6, -1)
    logits = head(h, g)
    out.update(head_h=h.numpy(), head_g=g.numpy(), head_w=head.w.weight.detach().numpy(),
               head_c=head.candidate.weight.detach().numpy(), head_gr=head.global_readout.weight.detach().numpy(),
               head_logits=logits.numpy())
    for temp in (1.0, 0.5, 2.0):
        out[f'probs_t{temp}'] = ref_probabilities(logits, temp).numpy()
    np.savez_compressed(OUT / 'ops.npz', **out)
    print('ops.npz', len(out), 'arrays')


if __name__ == '__main__':
    torch.manual_seed(0)
    op_level()
    end_to_end('tiny_config1', wl.TINY, 1, 0.0, wl.tiny_requests(1))
    end_to_end('tiny_gains', wl.TINY, 11, 0.1, wl.tiny_requests(11, eoi=None, requests=3, questions=2,
                                                               state=(20, 300)))
