"""The B200 modules inside the reference's own callers, with no reference source edited.

The reference package (oracle/_ref/, an unmodified copy made by oracle/make_ref.py) builds its
own JudgmentModel around a Hugging Face backbone; `install_b200_inference(model)` substitutes the
hot-path modules; then the reference's own code drives them in every execution mode it has:

  * serving:       model(request)             bongard/model.py:417-458 (encode, state_kv, decode_batch)
  * padded batch:  model([requests])          bongard/model.py:460-518 (encode_batch, state groups)
  * packed:        model.packing = True       bongard/packing.py:228-318 (forward_packed)
  * public call:   Predictor.predict(json)    bongard/inference.py:284-339

Ground truth is the fixture the reference produced in fp32 on CPU; the yardstick is the
reference's own bf16-vs-fp32 spread stored in the same fixture.
"""

import numpy as np
import pytest
import torch

from bongard_b200 import flash_varlen, packing, workload as wl
from bongard_b200.attention import B200DecoderAttention, B200EncoderAttention
from bongard_b200.install import install_b200_inference
from oracle import reference_math as om
from oracle import reference_package as rp

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not rp.available(), reason='oracle/_ref is absent: run python oracle/make_ref.py')]

DEV = 'cuda'


@pytest.fixture(scope='module')
def installed():
    ref = rp.load()
    compiler = rp.StubCompiler()
    model = rp.build_model(ref, wl.TINY, wl.make_weights(wl.TINY, 1), torch.bfloat16, DEV, compiler)
    counts = install_b200_inference(model)
    assert counts['encoder_attention'] == counts['decoder_attention'] == 2 and counts['mlp'] == 4
    assert model.packing_attention == 'b200'
    requests = wl.tiny_requests(1)
    return ref, model, compiler, requests, rp.to_reference_requests(ref, requests)


def probs(ref, result):
    return np.concatenate([ref.probabilities(v['logits'].float(), 1.0).numpy() for a in result for v in a.values()])


def bound(gold):
    """The model runs in bf16 with the residual adds, embeddings and state projections still executed
    by PyTorch in bf16 (the Hugging Face layer code owns them), so the yardstick is the reference's own
    bf16-vs-fp32 spread on this case, with a quarter of slack for a different summation order."""
    return 1.25 * max(float(np.abs(gold['probs_packed_fp32'] - gold['probs_packed_bf16']).max()), 1e-3)


def test_modules_are_substituted_in_the_reference_model(installed):
    _, model, _, _, _ = installed
    assert all(isinstance(l.self_attn, B200EncoderAttention) for l in model.backbone.encoder.text_model.layers)
    assert all(isinstance(l.self_attn, B200DecoderAttention) for l in model.backbone.decoder.layers)
    keys = set(model.state_dict())
    assert 'backbone.decoder.layers.0.self_attn.k_proj.weight' in keys      # native parameter names survive


@torch.inference_mode()
def test_serving_mode(installed, golden_dir):
    ref, model, _, _, ref_requests = installed
    gold = np.load(golden_dir / 'tiny_config1.npz')
    model.packing = False
    got = probs(ref, [model(r) for r in ref_requests])
    assert np.abs(got - gold['probs_serving_fp32']).max() <= bound(gold)


@torch.inference_mode()
def test_padded_batch_mode(installed, golden_dir):
    ref, model, _, _, ref_requests = installed
    gold = np.load(golden_dir / 'tiny_config1.npz')
    model.packing = False
    got = probs(ref, model(ref_requests))
    assert np.abs(got - gold['probs_serving_fp32']).max() <= bound(gold)


@torch.inference_mode()
def test_packed_mode_runs_the_reference_forward_packed(installed, golden_dir, monkeypatch):
    ref, model, _, _, ref_requests = installed
    gold = np.load(golden_dir / 'tiny_config1.npz')
    built = []
    native = packing.packed_layout
    monkeypatch.setattr(packing, 'packed_layout', lambda *a, **k: built.append(k.get('backend')) or native(*a, **k))
    model.packing = True
    try:
        got = probs(ref, model(ref_requests))
        # with a pack multiple the reference appends a dummy segment / dummy question (packing.py:243-252, 278-283)
        model.pack_multiple = 32
        padded = probs(ref, model(ref_requests))
        # two requests that share owner and state are encoded once (packing.py:232-238)
        twin = ref.Request(ref_requests[0].state, {'x': list(ref_requests[1].questions.values())[0]}, 0)
        shared = model([ref_requests[0], twin], state_owners=[0, 0])
    finally:
        model.packing = False
        del model.pack_multiple
    assert built and set(built) == {'b200'}          # the reference's forward_packed asked for, and got, B200 layouts
    assert np.abs(got - gold['probs_packed_fp32']).max() <= bound(gold)
    assert np.abs(padded - got).max() <= 2e-3
    assert set(shared[1]) == {'x'} and torch.isfinite(shared[1]['x']['logits']).all()


@torch.inference_mode()
def test_predictor_predict(installed, golden_dir):
    ref, model, compiler, requests, ref_requests = installed
    gold = np.load(golden_dir / 'tiny_config1.npz')
    model.packing = False
    predictor = ref.Predictor(model, model_id='tiny')
    got = []
    for i, (request, compiled) in enumerate(zip(requests, ref_requests)):
        compiler.register(f's{i}', compiled)
        reply = predictor.predict(rp.request_json(f's{i}', request))
        for qid, q in request.questions.items():
            got.extend(reply['answers'][qid]['probabilities'][key] for key in q.keys)
    assert np.abs(np.asarray(got) - gold['probs_serving_fp32']).max() <= bound(gold)
    # one question only: the reference takes its cache-free path (share_state_kv False, inference.py:308-310)
    single = ref.Request(ref_requests[0].state, dict(list(ref_requests[0].questions.items())[:1]), 0)
    compiler.register('single', single)
    qid, q = next(iter(requests[0].questions.items()))
    one = wl.Request(requests[0].state, {qid: q})
    reply = predictor.predict(rp.request_json('single', one))
    want = gold['probs_serving_fp32'][:len(q.keys)]
    assert np.abs(np.asarray([reply['answers'][qid]['probabilities'][k] for k in q.keys]) - want).max() <= bound(gold)


def test_prefix_op_with_the_layout_the_reference_builds():
    """bongard/flash_varlen.py:129-139 as the reference calls it on CUDA with backend 'flash': the
    state bank, and key_seqlens / key_indices from the reference's own packed_layout
    (bongard/packing.py:86-101), for eight questions that share one state and two on another;
    forward and backward against the oracle."""
    ref = rp.load()
    native_layout = getattr(ref.packing.packed_layout, 'native', ref.packing.packed_layout)
    hq, hkv, d = 4, 2, 64
    lengths = [17, 40, 9, 33, 25, 64, 12, 30, 21, 50]
    owners, state_lengths = [0] * 8 + [1] * 2, [150, 90]
    layout = native_layout(lengths, [None], torch.device(DEV), owners=owners, state_lengths=state_lengths, backend='flash')
    assert layout.key_indices is not None and not layout.masks
    t, ts = sum(lengths), sum(state_lengths)
    g = torch.Generator().manual_seed(9)
    q, k, v, dout = (torch.randn(t, h, d, generator=g).bfloat16() for h in (hq, hkv, hkv, hq))
    ck, cv = (torch.randn(ts, hkv, d, generator=g).bfloat16() for _ in range(2))
    leaves = [x.float().requires_grad_(True) for x in (q, k, v, ck, cv)]
    want, _ = om.varlen_attention(*leaves[:3], lengths, 0.125, None, cross=(leaves[3], leaves[4]), owners=owners,
                                  state_lengths=state_lengths)
    want.backward(dout.float())
    to4 = lambda x: x.to(DEV).transpose(0, 1)[None].contiguous().requires_grad_(True)   # noqa: E731  [1,H,T,D] leaves
    q4, k4, v4, ck4, cv4 = (to4(x) for x in (q, k, v, ck, cv))
    # the module-level surface with the reference's layout object, window inactive
    out = flash_varlen.attention(q4, k4, v4, layout, 0.125, None, (ck4, cv4))
    assert float((out[0].detach().transpose(0, 1).float().cpu() - want.detach()).abs().max()) < 2e-2
    out.backward(dout.to(DEV).transpose(0, 1)[None])
    for got, leaf in zip((q4.grad, k4.grad, v4.grad, ck4.grad, cv4.grad), leaves):
        got = got[0].transpose(0, 1).float().cpu()
        assert float((got - leaf.grad).abs().max()) < 2e-2 * (float(leaf.grad.abs().max()) + 1e-6)
    # the op itself, argument for argument
    dev = [x.to(DEV) for x in (q, k, v, ck, cv)]
    out3, lse = flash_varlen.flash_prefix_forward(*dev, layout.key_indices, layout.cu_seqlens, layout.key_seqlens, 0.125)
    assert float((out3.float().cpu() - want.detach()).abs().max()) < 2e-2
    grads = flash_varlen.flash_prefix_backward(*dev, layout.key_indices, layout.cu_seqlens, layout.key_seqlens, out3, lse,
                                               dout.to(DEV), 0.125)
    for got, leaf in zip(grads, leaves):
        assert float((got.float().cpu() - leaf.grad).abs().max()) < 2e-2 * (float(leaf.grad.abs().max()) + 1e-6)
