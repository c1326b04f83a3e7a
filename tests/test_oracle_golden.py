"""The CPU oracle against fixtures produced by the reference itself (tests/golden/make_golden.py)."""

import numpy as np
import pytest
import torch

from bongard_b200 import workload as wl
from oracle import reference_math as om


@pytest.fixture(scope='module')
def ops(golden_dir):
    return {k: torch.from_numpy(v) for k, v in np.load(golden_dir / 'ops.npz').items()}


def close(a, b, tol):
    assert a.shape == b.shape
    assert float((a.double() - b.double()).abs().max()) <= tol, float((a.double() - b.double()).abs().max())


def test_rmsnorm(ops):
    close(om.rmsnorm(ops['norm_x'], ops['norm_w']), ops['norm_y'], 1e-6)
    close(om.rmsnorm(ops['norm_x'].bfloat16(), ops['norm_w']).float(), ops['norm_y_bf16'], 0)


def test_embedding(ops):
    y = om.embed(ops['emb_ids'], ops['emb_table'], ops['emb_eoi'], 64, eoi_token=123)
    close(y, ops['emb_y'], 0)
    y = om.embed(ops['emb_ids'], ops['emb_table'].bfloat16(), ops['emb_eoi'].bfloat16(), 64, eoi_token=123)
    close(y.float(), ops['emb_y_bf16'], 0)


def test_qk_norm_rope(ops):
    hidden = ops['qk_hidden']
    q = om.linear(hidden, ops['qk_wq']).view(-1, 4, 64)
    k = om.linear(hidden, ops['qk_wk']).view(-1, 2, 64)
    cos, sin = om.rope_tables(ops['qk_positions'], 64, 1e4, torch.float32)
    close(cos, ops['qk_cos'], 1e-6)
    close(sin, ops['qk_sin'], 1e-6)
    qq, kk = om.qk_norm_rope(q, k, ops['qk_qnorm'], ops['qk_knorm'], cos, sin)
    close(qq, ops['qk_q'], 2e-6)
    close(kk, ops['qk_k'], 2e-6)
    v = om.linear(hidden, ops['qk_wv']).view(-1, 2, 64)
    _, sk = om.qk_norm_rope(q, k, ops['qk_qnorm'], ops['qk_knorm'], None, None)
    close(sk, ops['state_k'], 2e-6)
    close(v, ops['state_v'], 1e-6)


@pytest.mark.parametrize('window', [None, 4, 5, 16])
def test_encoder_attention(ops, window):
    out, _ = om.varlen_attention(ops['att_q'], ops['att_k'], ops['att_v'], ops['att_lengths'].tolist(), 0.125, window)
    close(out, ops[f'att_enc_w{window}'], 2e-6)


@pytest.mark.parametrize('window', [None, 4, 16])
def test_decoder_attention(ops, window):
    out, lse = om.varlen_attention(
        ops['att_q'], ops['att_k'], ops['att_v'], ops['att_lengths'].tolist(), 0.125, window,
        cross=(ops['att_ck'], ops['att_cv']), owners=ops['att_owners'].tolist(),
        state_lengths=ops['att_state_lengths'].tolist())
    close(out, ops[f'att_dec_w{window}'], 2e-6)
    if window is None:
        # the serving path's two-partition merge computes the same joint softmax
        close(out[5:22], ops['att_partition_seg1'], 2e-6)
        assert lse.shape == (4, out.shape[0])


def test_mlp(ops):
    close(om.geglu_mlp(ops['mlp_x'], ops['mlp_gate'], ops['mlp_up'], ops['mlp_down']), ops['mlp_y'], 2e-6)


def test_head_and_probabilities(ops):
    logits = om.judgment_head(ops['head_h'], ops['head_g'], ops['head_w'], ops['head_c'], ops['head_gr'])
    close(logits, ops['head_logits'], 1e-6)
    for temp in (1.0, 0.5, 2.0):
        close(om.probabilities(ops['head_logits'], temp), ops[f'probs_t{temp}'], 1e-15)


def test_fp8_block_quantisation_roundtrip():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 300, generator=g)
    q, inv = om.quantize_e4m3_block(x, 1, 128)
    assert q.dtype == torch.float8_e4m3fn and inv.shape == (5, 3)
    back = om.dequantize_block(q, inv, 1, 128)
    # E4M3 has 3 mantissa bits: relative step 2^-3, so half-step 1/16 of the block amax at most
    assert float((back - x).abs().max()) <= float(x.abs().max()) / 16 + 1e-6
    w = torch.randn(256, 300, generator=g) * 0.02
    y = om.linear_fp8_block128(x, w, torch.float32)
    ref = x @ w.t()
    assert float((y - ref).abs().max()) < 0.05 * float(ref.abs().max()) + 1e-3


@pytest.mark.parametrize('name,seed,norm_std,kwargs', [
    ('tiny_config1', 1, 0.0, {}),
    ('tiny_gains', 11, 0.1, dict(eoi=None, requests=3, questions=2, state=(20, 300))),
])
def test_end_to_end(golden_dir, name, seed, norm_std, kwargs):
    gold = np.load(golden_dir / f'{name}.npz')
    weights = wl.make_weights(wl.TINY, seed, norm_std=norm_std)
    checksum = float(sum(v.double().abs().sum() for v in weights.values()))
    assert abs(checksum - float(gold['weights_checksum'][0])) < 1e-6 * checksum
    requests = wl.tiny_requests(seed, **kwargs)
    with torch.inference_mode():
        result = om.forward_packed(weights, wl.TINY, requests, 8)
    logits = torch.cat([v['logits'] for answers in result for v in answers.values()])
    probs = torch.cat([om.probabilities(v['logits']) for answers in result for v in answers.values()])
    readouts = torch.cat([v['readouts'] for answers in result for v in answers.values()])
    close(logits, torch.from_numpy(gold['logits_packed_fp32']), 5e-6)
    close(logits, torch.from_numpy(gold['logits_serving_fp32']), 5e-6)
    close(probs, torch.from_numpy(gold['probs_packed_fp32']), 2e-6)
    close(readouts, torch.from_numpy(gold['readouts_packed_fp32']), 5e-5)
    # the oracle in bf16 must sit inside the reference's own bf16 spread
    with torch.inference_mode():
        result = om.forward_packed(weights, wl.TINY, requests, 8, dtype=torch.bfloat16)
    probs16 = torch.cat([om.probabilities(v['logits'].float()) for answers in result for v in answers.values()])
    spread = float(np.abs(gold['probs_packed_fp32'] - gold['probs_packed_bf16']).max())
    assert float((probs16 - torch.from_numpy(gold['probs_packed_fp32'])).abs().max()) <= 2 * spread + 1e-3
