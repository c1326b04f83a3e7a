"""The reference-shaped call surfaces: module substitution into the Hugging Face backbone and
the function-level entry points (flash_varlen.attention, project_qk, enable_* installers)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from bongard_b200 import flash_varlen, packing, workload as wl  # noqa: E402
from bongard_b200 import attention as b200_attention  # noqa: E402
from bongard_b200.engine import JudgmentEngine  # noqa: E402
from bongard_b200.float8_training import enable_float8  # noqa: E402
from bongard_b200.fused_mlp import B200FusedMLP, enable_fused_mlp  # noqa: E402
from bongard_b200.hf import PackedJudge, build_backbone  # noqa: E402
from bongard_b200.install import install_b200_inference  # noqa: E402
from bongard_b200.te_linear import B200Linear, B200MLP, enable_te_linear  # noqa: E402
from oracle import reference_math as om  # noqa: E402

DEV = 'cuda'


def probs_of(result):
    return torch.cat([om.probabilities(v['logits'].float()) for a in result for v in a.values()])


@pytest.fixture(scope='module')
def tiny():
    weights = wl.make_weights(wl.TINY, 1)
    return weights, wl.tiny_requests(1)


def test_module_substitution_matches_reference_fixture(golden_dir, tiny):
    weights, requests = tiny
    gold = np.load(golden_dir / 'tiny_config1.npz')
    backbone = build_backbone(wl.TINY, weights)
    counts = install_b200_inference(backbone)
    assert counts == dict(encoder_attention=2, decoder_attention=2, mlp=4, norms=2 * 2 * 6 + 2)
    names = set(backbone.state_dict())
    assert 'encoder.text_model.layers.0.self_attn.q_proj.weight' in names       # HF-shaped keys survive
    result = PackedJudge(backbone, weights).forward_packed(requests, 8)
    probs = probs_of(result)
    spread = float(np.abs(gold['probs_packed_fp32'] - gold['probs_packed_bf16']).max())
    err = float((probs - torch.from_numpy(gold['probs_packed_fp32'])).abs().max())
    assert err <= max(spread, 1e-3) * 1.25, (err, spread)
    engine = probs_of(JudgmentEngine(weights, wl.TINY, residual='bf16').forward_packed(requests, 8))
    assert float((probs - engine).abs().max()) < 2e-3


def test_padded_question_batch_matches_packed(tiny):
    """The serving path's padded decoder batch (QuestionLayout) and the packed path agree."""
    weights, requests = tiny
    backbone = build_backbone(wl.TINY, weights)
    install_b200_inference(backbone)
    judge = PackedJudge(backbone, weights)
    request = requests[0]
    with torch.inference_mode():
        state = judge.encode([request.state])
        cross = judge.state_kv(state)
        rows = [q.tokens for q in request.questions.values()]
        packed = judge.decode(rows, [0] * len(rows), [len(request.state)], state, cross)
        width = max(map(len, rows))
        ids = torch.tensor([list(r) + [0] * (width - len(r)) for r in rows], device=DEV)
        valid = torch.arange(width, device=DEV)[None, :] < torch.tensor([len(r) for r in rows], device=DEV)[:, None]
        positions = (valid.long().cumsum(-1) - 1).clamp_min(0)
        layout = b200_attention.QuestionLayout(valid, positions)
        decoder = backbone.decoder
        hidden = decoder.embed_tokens(ids)
        emb = {t: decoder.rotary_emb(hidden, positions, t) for t in set(decoder.config.layer_types)}
        empty = torch.empty(0, device=DEV)
        for index, layer in enumerate(decoder.layers):
            hidden = layer(hidden, emb[decoder.config.layer_types[index]], empty, positions, None, False, state,
                           question_layout=layout, packed_cross=cross[index])
        hidden = decoder.norm(hidden)
    offset = 0
    for i, r in enumerate(rows):
        a, b = hidden[i, :len(r)].float(), packed[offset:offset + len(r)].float()
        assert float((a - b).abs().max()) <= 2e-2 + 1e-2 * float(b.abs().max())
        offset += len(r)


@pytest.mark.parametrize('window', [None, 4, 16])
def test_flash_varlen_attention_surface(golden_dir, window):
    """bongard.flash_varlen.attention's signature, [1,H,T,D] tensors, incl. an ACTIVE window."""
    g = {k: torch.from_numpy(v) for k, v in np.load(golden_dir / 'ops.npz').items() if k.startswith('att_')}
    to = lambda t: t.bfloat16().to(DEV).transpose(0, 1)[None].contiguous()   # noqa: E731  [T,H,D] -> [1,H,T,D]
    q, k, v, ck, cv = (to(g[n]) for n in ('att_q', 'att_k', 'att_v', 'att_ck', 'att_cv'))
    lengths = g['att_lengths'].tolist()
    layout = packing.packed_layout(lengths, [window], DEV)
    out = flash_varlen.attention(q, k, v, layout, 0.125, window)
    assert out.shape == q.shape
    want = g[f'att_enc_w{window}']
    assert float((out[0].transpose(0, 1).float().cpu() - want).abs().max()) < 4e-2
    layout = packing.packed_layout(lengths, [window], DEV, owners=g['att_owners'].tolist(),
                                   state_lengths=g['att_state_lengths'].tolist())
    out = packing.layout_attention(q, k, v, layout, 0.125, window, (ck, cv))
    want = g[f'att_dec_w{window}']
    assert float((out[0].transpose(0, 1).float().cpu() - want).abs().max()) < 4e-2
    with pytest.raises(ValueError):
        packing.layout_attention(q, k, v, layout, 0.125, window, (ck, cv), dropout=0.1)
    with pytest.raises(ValueError):
        packing.packed_layout(lengths, [window], DEV, backend='triton')


def test_custom_ops_keep_the_reference_contract():
    t, hq, hkv, d = 50, 4, 2, 64
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(t, h, d, generator=g).bfloat16().to(DEV) for h in (hq, hkv, hkv))
    cu = torch.tensor([0, 20, 50], dtype=torch.int32, device=DEV)
    out, lse = flash_varlen.flash_packed_forward(q, k, v, cu, cu, 0.125, False)
    assert out.shape == q.shape and lse.shape == (hq, t) and lse.dtype == torch.float32
    want, want_lse = om.varlen_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), [20, 30], 0.125, None)
    assert float((out.float().cpu() - want).abs().max()) < 2e-2
    assert float((lse.cpu() - want_lse).abs().max()) < 2e-2
    if flash_varlen.REGISTERED:
        out2, _ = torch.ops.bongard.flash_packed_forward(q, k, v, cu, cu, 0.125, False)
        assert torch.equal(out2, out)


def test_attention_surface_is_differentiable():
    """flash_varlen.attention / packing.layout_attention record a backward (encoder with an active
    window, decoder with a state prefix), and the custom ops carry the reference's autograd
    registration (bongard/flash_varlen.py:46-58, 113-126)."""
    hq, hkv, d, lengths, window = 4, 2, 64, [90, 37, 200], 64
    t = sum(lengths)
    g = torch.Generator().manual_seed(3)
    q, k, v, dout = (torch.randn(t, h, d, generator=g).bfloat16() for h in (hq, hkv, hkv, hq))

    def oracle(cross=None, owners=None, state_lengths=None, win=window):
        leaves = [x.float().requires_grad_(True) for x in (q, k, v)] + [x.float().requires_grad_(True) for x in cross or ()]
        out, _ = om.varlen_attention(*leaves[:3], lengths, 0.125, win, cross=tuple(leaves[3:]) or None, owners=owners,
                                     state_lengths=state_lengths)
        out.backward(dout.float())
        return [x.grad for x in leaves]

    def close(got, want):
        got, want = got.float().cpu(), want.float()
        assert float((got - want).abs().max()) < 2e-2 * (float(want.abs().max()) + 1e-6)

    to = lambda x: x.to(DEV).transpose(0, 1)[None].contiguous().requires_grad_(True)   # noqa: E731  [1,H,T,D] leaves
    q4, k4, v4 = to(q), to(k), to(v)
    layout = packing.packed_layout(lengths, [window], DEV)
    out = flash_varlen.attention(q4, k4, v4, layout, 0.125, window)
    out.backward(dout.to(DEV).transpose(0, 1)[None])
    for got, want in zip((q4.grad, k4.grad, v4.grad), oracle()):
        close(got[0].transpose(0, 1), want)

    state_lengths, owners = [70, 130], [0, 0, 1]
    ck, cv = (torch.randn(sum(state_lengths), hkv, d, generator=g).bfloat16() for _ in range(2))
    q4, k4, v4, ck4, cv4 = to(q), to(k), to(v), to(ck), to(cv)
    layout = packing.packed_layout(lengths, [window], DEV, owners=owners, state_lengths=state_lengths)
    out = packing.layout_attention(q4, k4, v4, layout, 0.125, window, (ck4, cv4))
    out.backward(dout.to(DEV).transpose(0, 1)[None])
    for got, want in zip((q4.grad, k4.grad, v4.grad, ck4.grad, cv4.grad), oracle((ck, cv), owners, state_lengths)):
        close(got[0].transpose(0, 1), want)

    if flash_varlen.REGISTERED:
        cu = torch.tensor([0, 90, 127, 327], dtype=torch.int32, device=DEV)
        leaves = [x.to(DEV).requires_grad_(True) for x in (q, k, v)]
        out, _ = torch.ops.bongard.flash_packed_forward(*leaves, cu, cu, 0.125, False)
        out.backward(dout.to(DEV))
        for leaf, want in zip(leaves, oracle(win=None)):
            close(leaf.grad, want)
        # an empty gather: one private state per question, back to back
        states = [50, 64, 20]
        ck, cv = (torch.randn(sum(states), hkv, d, generator=g).bfloat16() for _ in range(2))
        cuk = torch.tensor([0, 140, 241, 461], dtype=torch.int32, device=DEV)
        leaves = [x.to(DEV).requires_grad_(True) for x in (q, k, v, ck, cv)]
        out, _ = torch.ops.bongard.flash_prefix_forward(*leaves, torch.zeros(0, dtype=torch.int64, device=DEV), cu, cuk, 0.125)
        out.backward(dout.to(DEV))
        for leaf, want in zip(leaves, oracle((ck, cv), [0, 1, 2], states, win=None)):
            close(leaf.grad, want)


def reference_gather(lengths, owners, state_lengths):
    """key_seqlens and key_indices as the reference's packed_layout builds them
    (bongard/packing.py:86-101): per question its owner's state rows, then its own rows, as
    indices into cat(state bank, own keys)."""
    from itertools import accumulate

    state_offsets = list(accumulate(state_lengths, initial=0))
    query_offsets = list(accumulate(lengths, initial=0))
    total = sum(state_lengths)
    indices = []
    for i, owner in enumerate(owners):
        indices.extend(range(state_offsets[owner], state_offsets[owner + 1]))
        indices.extend(range(total + query_offsets[i], total + query_offsets[i + 1]))
    key_cu = list(accumulate((state_lengths[o] + n for o, n in zip(owners, lengths)), initial=0))
    return (torch.tensor(key_cu, dtype=torch.int32, device=DEV), torch.tensor(indices, device=DEV),
            torch.tensor(query_offsets, dtype=torch.int32, device=DEV))


def test_prefix_ops_take_the_state_bank_and_the_gather():
    """The prefix ops with the reference's own arguments (bongard/flash_varlen.py:129-139): ck/cv
    are the state BANK - one state per owner, shared by its questions - and `indices` is the
    gather over cat(bank, own keys).  Eight questions on one state plus two on another, forward
    and backward against the oracle; state rows nobody reads keep a zero gradient."""
    hq, hkv, d = 4, 2, 64
    lengths = [17, 40, 9, 33, 25, 64, 12, 30, 21, 50]
    owners = [0] * 8 + [2] * 2
    state_lengths = [150, 70, 90]             # state 1 belongs to nobody in this group
    t, ts = sum(lengths), sum(state_lengths)
    g = torch.Generator().manual_seed(8)
    q, k, v, dout = (torch.randn(t, h, d, generator=g).bfloat16() for h in (hq, hkv, hkv, hq))
    ck, cv = (torch.randn(ts, hkv, d, generator=g).bfloat16() for _ in range(2))
    cuk, indices, cuq = reference_gather(lengths, owners, state_lengths)
    leaves = [x.float().requires_grad_(True) for x in (q, k, v, ck, cv)]
    want, want_lse = om.varlen_attention(*leaves[:3], lengths, 0.125, None, cross=(leaves[3], leaves[4]), owners=owners,
                                         state_lengths=state_lengths)
    want.backward(dout.float())
    dev = [x.to(DEV) for x in (q, k, v, ck, cv)]
    out, lse = flash_varlen.flash_prefix_forward(*dev, indices, cuq, cuk, 0.125)
    assert out.shape == q.shape and lse.shape == (hq, t)
    assert float((out.float().cpu() - want.detach()).abs().max()) < 2e-2
    assert float((lse.cpu() - want_lse.detach()).abs().max()) < 2e-2
    grads = flash_varlen.flash_prefix_backward(*dev, indices, cuq, cuk, out, lse, dout.to(DEV), 0.125)
    for got, leaf in zip(grads, leaves):
        assert got.shape == leaf.shape
        assert float((got.float().cpu() - leaf.grad).abs().max()) < 2e-2 * (float(leaf.grad.abs().max()) + 1e-6)
    assert not grads[3][150:220].any() and not grads[4][150:220].any()
    if flash_varlen.REGISTERED:
        out2, _ = torch.ops.bongard.flash_prefix_forward(*dev, indices, cuq, cuk, 0.125)
        assert torch.equal(out2, out)
    # a gather that is not [state run | own run], or that runs past the bank, is refused on the host
    with pytest.raises(ValueError):
        flash_varlen.flash_prefix_forward(*dev, indices.flip(0), cuq, cuk, 0.125)
    with pytest.raises(ValueError):
        flash_varlen.flash_prefix_forward(dev[0], dev[1], dev[2], dev[3][:100], dev[4][:100], indices, cuq, cuk, 0.125)


def test_converted_mlp_trains_like_the_native_one(tiny):
    """Train mode: the converted MLP (te_linear and fused_mlp surfaces, bf16 recipe) gives the native
    module's gradients for its input and its weights; the fp8 recipe refuses to train."""
    weights, _ = tiny
    x = torch.randn(3, 50, wl.TINY.hidden, generator=torch.Generator().manual_seed(4)).bfloat16().to(DEV)
    dy = torch.randn(3, 50, wl.TINY.hidden, generator=torch.Generator().manual_seed(5)).bfloat16().to(DEV)

    def run(convert):
        backbone = build_backbone(wl.TINY, weights).train()
        layer = backbone.decoder.layers[0]
        convert(backbone)
        inp = x.clone().requires_grad_(True)
        out = layer.mlp(layer.pre_feedforward_layernorm(inp))
        out.backward(dy)
        grads = {n: p.grad.float().cpu() for n, p in layer.named_parameters() if p.grad is not None}
        return out.detach().float().cpu(), inp.grad.float().cpu(), grads

    want_out, want_dx, want = run(lambda b: None)
    for convert in (lambda b: enable_te_linear(b, mlp='bf16'), lambda b: enable_fused_mlp(b, 'bf16')):
        out, dx, grads = run(convert)
        assert float((out - want_out).abs().max()) < 3e-2 * float(want_out.abs().max()) + 1e-3
        assert float((dx - want_dx).abs().max()) < 3e-2 * float(want_dx.abs().max()) + 1e-3
        down = next(v for k, v in grads.items() if 'down' in k)
        assert float((down - want['mlp.down_proj.weight']).abs().max()) < 3e-2 * float(want['mlp.down_proj.weight'].abs().max())
        if 'mlp.layer_norm_weight' in grads:      # the fused module owns the pre-norm: its gain gradient comes from the norm-backward kernel
            gain = want['pre_feedforward_layernorm.weight']
            assert float((grads['mlp.layer_norm_weight'] - gain).abs().max()) < 3e-2 * float(gain.abs().max())
    backbone = build_backbone(wl.TINY, weights).train()
    enable_te_linear(backbone, mlp='fp8')
    with pytest.raises(ValueError, match='forward-only'):
        backbone.decoder.layers[0].mlp(x.clone().requires_grad_(True))


def test_project_qk_surface(golden_dir, tiny):
    weights, _ = tiny
    g = {k: torch.from_numpy(v) for k, v in np.load(golden_dir / 'ops.npz').items() if k.startswith(('qk_', 'state_'))}
    backbone = build_backbone(wl.TINY, weights)
    attn = backbone.encoder.text_model.layers[0].self_attn
    with torch.no_grad():
        attn.q_proj.weight.copy_(g['qk_wq']); attn.k_proj.weight.copy_(g['qk_wk'])      # noqa: E702
        attn.q_norm.weight.copy_(g['qk_qnorm']); attn.k_norm.weight.copy_(g['qk_knorm'])  # noqa: E702
    hidden = g['qk_hidden'].bfloat16().to(DEV)[None]
    pe = (g['qk_cos'].bfloat16().to(DEV)[None], g['qk_sin'].bfloat16().to(DEV)[None])
    with torch.no_grad():
        q, k = b200_attention.project_qk(attn, hidden, pe, 'b200')
    assert q.shape == (1, 4, hidden.shape[1], 64) and k.shape == (1, 2, hidden.shape[1], 64)
    assert float((q[0].transpose(0, 1).float().cpu() - g['qk_q']).abs().max()) < 6e-2
    assert float((k[0].transpose(0, 1).float().cpu() - g['qk_k']).abs().max()) < 6e-2


def test_enable_surfaces_and_fp8_end_to_end(tiny):
    weights, requests = tiny
    backbone = build_backbone(wl.TINY, weights)
    assert enable_fused_mlp(backbone, 'bf16') == 4
    assert isinstance(backbone.decoder.layers[0].mlp, B200FusedMLP)
    assert isinstance(backbone.decoder.layers[0].pre_feedforward_layernorm, torch.nn.Identity)
    with pytest.raises(ValueError):
        enable_fused_mlp(backbone, 'nvfp4')
    backbone = build_backbone(wl.TINY, weights)
    assert enable_te_linear(backbone, mlp='bf16', attention='bf16') == {'mlp': 4, 'attention': 16}
    assert isinstance(backbone.encoder.text_model.layers[0].mlp, B200MLP)
    assert isinstance(backbone.encoder.text_model.layers[0].self_attn.o_proj, B200Linear)
    with pytest.raises(ValueError):
        enable_te_linear(backbone)
    # FP8 everywhere: module path and engine agree with each other and stay near the bf16 result
    backbone = build_backbone(wl.TINY, weights)
    assert enable_float8(backbone, 'block128') == 2 * 2 * 7
    install_b200_inference(backbone, linears='fp8')
    p_mod = probs_of(PackedJudge(backbone, weights).forward_packed(requests, 8))
    # the substituted modules run the reference's bf16 chain: compare with the engine in the same mode
    p_eng = probs_of(JudgmentEngine(weights, wl.TINY, linears='fp8', residual='bf16').forward_packed(requests, 8))
    p_bf16 = probs_of(JudgmentEngine(weights, wl.TINY, residual='bf16').forward_packed(requests, 8))
    assert float((p_mod - p_eng).abs().max()) < 5e-3
    assert float((p_eng - p_bf16).abs().max()) < 3e-2
    with pytest.raises(ValueError):
        enable_float8(backbone, 'tensorwise')


def test_padded_dense_encoder_batch_matches_packed(tiny):
    """The reference's encode_batch path: a right-padded [B, S] batch with an attention mask."""
    weights, requests = tiny
    backbone = build_backbone(wl.TINY, weights)
    install_b200_inference(backbone)
    states = [r.state for r in requests[:3]]
    packed = PackedJudge(backbone, weights).encode(states)[0]
    width = max(map(len, states))
    ids = torch.tensor([list(st) + [0] * (width - len(st)) for st in states], device=DEV)
    lengths = torch.tensor([len(st) for st in states], device=DEV)
    mask = (torch.arange(width, device=DEV)[None, :] < lengths[:, None]).long()
    with torch.inference_mode():
        dense = backbone.encoder(input_ids=ids, attention_mask=mask, bongard_encoder_windows={}, use_cache=False).last_hidden_state
    offset = 0
    for i, st in enumerate(states):
        a, b = dense[i, :len(st)].float(), packed[offset:offset + len(st)].float()
        assert float((a - b).abs().max()) <= 3e-2 + 2e-2 * float(b.abs().max())
        offset += len(st)


def test_substituted_norm_and_qk_norm_rope_are_differentiable(tiny):
    """The substituted RMSNorm and the fused QK-norm + RoPE surface record their backward kernels: gradients
    for the input and the gains agree with the native modules / the fp32 oracle."""
    weights, _ = tiny
    backbone = build_backbone(wl.TINY, weights).train()
    native = backbone.decoder.layers[0].pre_self_attn_layernorm
    with torch.no_grad():
        native.weight.normal_(0, 0.2, generator=torch.Generator(device=DEV).manual_seed(1))
    x = torch.randn(2, 70, wl.TINY.hidden, generator=torch.Generator().manual_seed(6)).bfloat16().to(DEV)
    dy = torch.randn(2, 70, wl.TINY.hidden, generator=torch.Generator().manual_seed(7)).bfloat16().to(DEV)

    def grads(module):
        module.zero_grad()
        inp = x.clone().requires_grad_(True)
        module(inp).backward(dy)
        return inp.grad.float().cpu(), module.weight.grad.float().cpu()

    want_dx, want_dw = grads(native)
    got_dx, got_dw = grads(b200_attention.B200RMSNorm(native))
    assert float((got_dx - want_dx).abs().max()) < 2e-2 * float(want_dx.abs().max()) + 1e-3
    assert float((got_dw - want_dw).abs().max()) < 2e-2 * float(want_dw.abs().max()) + 1e-3
    with torch.no_grad():                         # inference keeps the plain kernel and records nothing
        assert not b200_attention.B200RMSNorm(native)(x).requires_grad

    attn = backbone.encoder.text_model.layers[0].self_attn
    d, hq, hkv, l = wl.TINY.head_dim, wl.TINY.q_heads, wl.TINY.kv_heads, 90
    gen = torch.Generator().manual_seed(8)
    q = torch.randn(1, l, hq, d, generator=gen).bfloat16()
    k = torch.randn(1, l, hkv, d, generator=gen).bfloat16()
    dq, dk = torch.randn(1, hq, l, d, generator=gen).bfloat16(), torch.randn(1, hkv, l, d, generator=gen).bfloat16()
    cos, sin = om.rope_tables(torch.arange(l), d, 1e4, torch.bfloat16)
    qd, kd = q.to(DEV).requires_grad_(True), k.to(DEV).requires_grad_(True)
    attn.zero_grad()
    oq, ok = b200_attention.qk_norm_rope(qd, kd, attn.q_norm, attn.k_norm, (cos.to(DEV)[None], sin.to(DEV)[None]))
    torch.autograd.backward([oq, ok], [dq.to(DEV), dk.to(DEV)])
    qf, kf = q[0].float().requires_grad_(True), k[0].float().requires_grad_(True)
    qw, kw = (n.weight.detach().float().cpu().requires_grad_(True) for n in (attn.q_norm, attn.k_norm))
    wq, wk = om.qk_norm_rope(qf, kf, qw, kw, cos.float(), sin.float())
    torch.autograd.backward([wq, wk], [dq[0].transpose(0, 1).float(), dk[0].transpose(0, 1).float()])
    for got, want in ((qd.grad[0], qf.grad), (kd.grad[0], kf.grad), (attn.q_norm.weight.grad, qw.grad),
                      (attn.k_norm.weight.grad, kw.grad)):
        assert float((got.float().cpu() - want).abs().max()) < 2e-2 * float(want.abs().max()) + 2e-3


@pytest.mark.parametrize('decoder', [False, True])
@pytest.mark.parametrize('layer_index', [0, 1])
def test_packed_attention_module_trains(tiny, decoder, layer_index):
    """With gradients enabled the substituted attention modules run their projections, QK-norm + RoPE
    and the packed attention through the backward kernels: gradients of the input, of every projection,
    of the QK gains and (decoder) of the shared state K/V against autograd of the fp32 oracle."""
    weights, _ = tiny
    shape = wl.TINY
    backbone = build_backbone(shape, weights).train()
    install_b200_inference(backbone)
    stack = backbone.decoder if decoder else backbone.encoder.text_model
    module = stack.layers[layer_index].self_attn
    with torch.no_grad():
        for norm, seed in ((module.q_norm, 1), (module.k_norm, 2)):
            norm.weight.normal_(0, 0.2, generator=torch.Generator(device=DEV).manual_seed(seed))
    lengths = [70, 200, 33]
    t = sum(lengths)
    gen = torch.Generator().manual_seed(11 + layer_index)
    hidden = torch.randn(t, shape.hidden, generator=gen).bfloat16()
    dout = torch.randn(t, shape.hidden, generator=gen).bfloat16()
    owners, state_lengths = [1, 1, 0], [90, 150]      # questions of one owner are consecutive (backward plan)
    ck = torch.randn(sum(state_lengths), shape.kv_heads, shape.head_dim, generator=gen).bfloat16()
    cv = torch.randn(sum(state_lengths), shape.kv_heads, shape.head_dim, generator=gen).bfloat16()

    module.zero_grad()
    hd = hidden.to(DEV).requires_grad_(True)
    if decoder:
        layout = packing.packed_layout(lengths, [], DEV, owners=owners, state_lengths=state_lengths)
        ckd, cvd = ck.to(DEV).requires_grad_(True), cv.to(DEV).requires_grad_(True)
        out = packing.decoder_attention(module, hd[None], None, None, layout, (ckd, cvd))[0]
    else:
        layout = packing.packed_layout(lengths, [], DEV)
        out = packing.encoder_attention(module, hd[None], None, layout)[0]
    out.backward(dout.to(DEV)[None])

    leaf = lambda v: v.detach().float().cpu().requires_grad_(True)
    hf_, wq, wk, wv, wo = leaf(hidden), leaf(module.q_proj.weight), leaf(module.k_proj.weight), leaf(module.v_proj.weight), leaf(module.o_proj.weight)
    gq, gk = leaf(module.q_norm.weight), leaf(module.k_norm.weight)
    ckf, cvf = leaf(ck), leaf(cv)
    q = om.linear(hf_, wq).view(t, shape.q_heads, shape.head_dim)
    k = om.linear(hf_, wk).view(t, shape.kv_heads, shape.head_dim)
    v = om.linear(hf_, wv).view(t, shape.kv_heads, shape.head_dim)
    positions = torch.cat([torch.arange(n) for n in lengths])
    cos, sin = om.rope_tables(positions, shape.head_dim, shape.layer_theta(layer_index), torch.float32)
    q, k = om.qk_norm_rope(q, k, gq, gk, cos, sin, shape.eps)
    window = shape.layer_window(layer_index)
    if decoder:
        attended, _ = om.varlen_attention(q, k, v, lengths, shape.scale, window, cross=(ckf, cvf), owners=owners,
                                          state_lengths=state_lengths)
    else:
        attended, _ = om.varlen_attention(q, k, v, lengths, shape.scale, window)
    want = om.linear(attended.reshape(t, -1), wo)
    want.backward(dout.float())

    def close(got, ref, what):
        got, ref = got.detach().float().cpu().reshape(ref.shape), ref.detach()
        err, scale = float((got - ref).abs().max()), float(ref.abs().max())
        assert err < 4e-2 * scale + 2e-3, (what, err, scale)

    close(out[0], want, 'out')
    close(hd.grad, hf_.grad, 'dhidden')
    for name, ref in (('q_proj', wq), ('k_proj', wk), ('v_proj', wv), ('o_proj', wo)):
        close(getattr(module, name).weight.grad, ref.grad, name)
    close(module.q_norm.weight.grad, gq.grad, 'q gain')
    close(module.k_norm.weight.grad, gk.grad, 'k gain')
    if decoder:
        close(ckd.grad, ckf.grad, 'state k')
        close(cvd.grad, cvf.grad, 'state v')


def test_substituted_encoder_trains_like_the_native_one(tiny):
    """Whole encoder, train mode: the backbone with every hot-path module substituted, driven packed, gives
    the native backbone's parameter gradients (native: one dense sequence at a time, PyTorch autograd)."""
    weights, _ = tiny
    shape = wl.TINY
    lengths = [70, 200]
    gen = torch.Generator().manual_seed(21)
    ids = [torch.randint(2, shape.vocab, (n,), generator=gen) for n in lengths]
    dys = [torch.randn(n, shape.hidden, generator=gen).bfloat16().to(DEV) for n in lengths]

    native = build_backbone(shape, weights).train()
    for tokens, dy in zip(ids, dys):
        out = native.encoder(input_ids=tokens.to(DEV)[None], use_cache=False).last_hidden_state
        (out[0].float() * dy.float()).sum().backward()
    want = {n: p.grad.float().cpu() for n, p in native.encoder.named_parameters() if p.grad is not None}

    ours = build_backbone(shape, weights).train()
    install_b200_inference(ours)
    layout = packing.packed_layout(lengths, [], DEV)
    empty = torch.empty(0, device=DEV)
    out = ours.encoder(input_ids=torch.cat(ids).to(DEV)[None], position_ids=layout.positions,
                       attention_mask={'full_attention': empty, 'sliding_attention': empty}, packed_layout=layout,
                       use_cache=False).last_hidden_state
    (out[0].float() * torch.cat(dys).float()).sum().backward()
    got = {n: p.grad.float().cpu() for n, p in ours.encoder.named_parameters() if p.grad is not None}
    # the converted MLP stacks gate and up into one trainable weight: back to the Hugging Face names
    for name in [n for n in got if n.endswith('mlp.gate_up.weight')]:
        layer = name[:-len('gate_up.weight')]
        got[layer + 'gate_proj.weight'], got[layer + 'up_proj.weight'] = got[name].split(shape.intermediate)
        got[layer + 'down_proj.weight'] = got[layer + 'down.weight']

    checked = 0
    for name, ref in want.items():
        if 'vision' in name or float(ref.abs().max()) == 0:
            continue
        assert name in got, (name, sorted(got))
        err, scale = float((got[name] - ref).abs().max()), float(ref.abs().max())
        assert err < 6e-2 * scale + 1e-3, (name, err, scale)
        checked += 1
    assert checked >= 2 * 11       # per layer: 4 projections, 2 QK gains, 3 MLP weights, 4 norms (some tied names aside)


def test_state_projection_trains(tiny):
    """The decoder's shared state K/V (bongard/model.py:135-139 project_state_kv: K = k_norm(k_proj(state)) without
    rotation, V = v_proj(state)) is differentiable in train mode: state, both projections and the key gain."""
    weights, _ = tiny
    shape = wl.TINY
    backbone = build_backbone(shape, weights).train()
    install_b200_inference(backbone)
    module = backbone.decoder.layers[1].self_attn
    with torch.no_grad():
        module.k_norm.weight.normal_(0, 0.2, generator=torch.Generator(device=DEV).manual_seed(3))
    gen = torch.Generator().manual_seed(31)
    s = 150
    state = torch.randn(1, s, shape.hidden, generator=gen).bfloat16()
    dk = torch.randn(1, shape.kv_heads, s, shape.head_dim, generator=gen).bfloat16()
    dv = torch.randn(1, shape.kv_heads, s, shape.head_dim, generator=gen).bfloat16()
    module.zero_grad()
    sd = state.to(DEV).requires_grad_(True)
    keys, values = module._cross(None, sd, None)
    torch.autograd.backward([keys, values], [dk.to(DEV), dv.to(DEV)])
    with torch.no_grad():
        keys_inference, values_inference = module._cross(None, state.to(DEV), None)
    assert float((keys - keys_inference).abs().max()) < 2e-2 and torch.equal(values, values_inference)

    leaf = lambda v: v.detach().float().cpu().requires_grad_(True)
    sf, wk, wv, gk = leaf(state), leaf(module.k_proj.weight), leaf(module.v_proj.weight), leaf(module.k_norm.weight)
    k = om.rmsnorm(om.linear(sf[0], wk).view(s, shape.kv_heads, shape.head_dim), gk, shape.eps)
    v = om.linear(sf[0], wv).view(s, shape.kv_heads, shape.head_dim)
    torch.autograd.backward([k, v], [dk[0].transpose(0, 1).float(), dv[0].transpose(0, 1).float()])
    for got, ref, what in ((sd.grad, sf.grad, 'state'), (module.k_proj.weight.grad, wk.grad, 'k_proj'),
                           (module.v_proj.weight.grad, wv.grad, 'v_proj'), (module.k_norm.weight.grad, gk.grad, 'k gain')):
        got = got.float().cpu().reshape(ref.shape)
        err, scale = float((got - ref).abs().max()), float(ref.abs().max())
        assert err < 4e-2 * scale + 2e-3, (what, err, scale)


def test_substituted_decoder_trains_like_the_native_one(tiny):
    """Whole decoder, train mode: questions packed over two shared states, the state K/V projected per layer by
    the substituted module, against the native decoder run one question at a time on its own state: gradients of
    every decoder parameter and of the encoder states."""
    weights, _ = tiny
    shape = wl.TINY
    state_lengths, lengths, owners = [90, 150], [40, 25, 33], [0, 0, 1]
    gen = torch.Generator().manual_seed(41)
    states = [torch.randn(n, shape.hidden, generator=gen).bfloat16() for n in state_lengths]
    ids = [torch.randint(2, shape.vocab, (n,), generator=gen) for n in lengths]
    dys = [torch.randn(n, shape.hidden, generator=gen).bfloat16().to(DEV) for n in lengths]

    native = build_backbone(shape, weights).train()
    native_states = [s.to(DEV).requires_grad_(True) for s in states]
    for tokens, dy, owner in zip(ids, dys, owners):
        out = native.decoder(input_ids=tokens.to(DEV)[None], encoder_hidden_states=native_states[owner][None],
                             use_cache=False).last_hidden_state
        (out[0].float() * dy.float()).sum().backward()
    want = {n: p.grad.float().cpu() for n, p in native.decoder.named_parameters() if p.grad is not None}

    ours = build_backbone(shape, weights).train()
    install_b200_inference(ours)
    decoder = ours.decoder
    our_states = [s.to(DEV).requires_grad_(True) for s in states]
    layout = packing.packed_layout(lengths, [], DEV, owners=owners, state_lengths=state_lengths)
    hidden = decoder.embed_tokens(torch.cat(ids).to(DEV)[None])
    embeddings = {t: decoder.rotary_emb(hidden, layout.positions, t) for t in set(decoder.config.layer_types)}
    empty = torch.empty(0, device=DEV)
    for index, layer in enumerate(decoder.layers):
        parts = [layer.self_attn._cross(None, s[None], None) for s in our_states]
        cross = (torch.cat([k[0].transpose(0, 1) for k, _ in parts]), torch.cat([v[0].transpose(0, 1) for _, v in parts]))
        hidden = layer(hidden, embeddings[decoder.config.layer_types[index]], empty, layout.positions, None, False,
                       None, question_layout=layout, packed_cross=cross)
    out = decoder.norm(hidden)[0]
    (out.float() * torch.cat(dys).float()).sum().backward()
    got = {n: p.grad.float().cpu() for n, p in decoder.named_parameters() if p.grad is not None}
    for name in [n for n in got if n.endswith('mlp.gate_up.weight')]:
        layer = name[:-len('gate_up.weight')]
        got[layer + 'gate_proj.weight'], got[layer + 'up_proj.weight'] = got[name].split(shape.intermediate)
        got[layer + 'down_proj.weight'] = got[layer + 'down.weight']

    checked = 0
    for name, ref in want.items():
        if float(ref.abs().max()) == 0:
            continue
        assert name in got, (name, sorted(got))
        err, scale = float((got[name] - ref).abs().max()), float(ref.abs().max())
        assert err < 6e-2 * scale + 1e-3, (name, err, scale)
        checked += 1
    assert checked >= 2 * 11
    for mine, theirs in zip(our_states, native_states):
        err, scale = float((mine.grad.float() - theirs.grad.float()).abs().max()), float(theirs.grad.float().abs().max())
        assert err < 6e-2 * scale + 1e-3, ('state', err, scale)
