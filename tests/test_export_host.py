"""Export inverses with the reference's signatures (bongard/fused_mlp.py:101-124 hf_state_dict(backbone),
bongard/te_linear.py:144-161 restore_hf_layout(backbone, state)): a converted backbone's state comes back
under Hugging Face keys with the original tensors, and survives a checkpoint round trip.  CPU only: the
conversions are built without the device check and no kernel runs."""

import pytest
import torch

from bongard_b200 import checkpoint, fused_mlp, te_linear, workload as wl
from bongard_b200.hf import build_backbone


def convert(backbone, how):
    for layer in list(backbone.encoder.text_model.layers) + list(backbone.decoder.layers):
        if how == 'te':
            layer.mlp = te_linear.B200MLP(layer.mlp)
            for name in te_linear.ATTENTION_PROJECTIONS:
                setattr(layer.self_attn, name, te_linear.B200Linear([getattr(layer.self_attn, name)]))
        else:
            layer.mlp = fused_mlp.B200FusedMLP(layer.mlp, layer.pre_feedforward_layernorm)
            layer.pre_feedforward_layernorm = torch.nn.Identity()


@pytest.mark.parametrize('how', ['te', 'fused'])
def test_converted_backbone_exports_hugging_face_keys(how, tmp_path):
    weights = wl.make_weights(wl.TINY, 2, norm_std=0.1, dtype=torch.bfloat16)
    backbone = build_backbone(wl.TINY, weights, device='cpu')
    assert fused_mlp.hf_state_dict(backbone) is None                 # nothing converted: the caller saves as is
    native = {k: v.clone() for k, v in backbone.state_dict().items()}
    convert(backbone, how)
    converted = set(backbone.state_dict())
    assert any('gate_up' in k for k in converted) and not any('gate_proj' in k for k in converted)
    state = fused_mlp.hf_state_dict(backbone)
    assert set(state) == set(native)
    assert all(torch.equal(state[k], native[k]) for k in native)
    # the reference's own save path hands this state to save_pretrained (bongard/model.py:531-539);
    # the checkpoint loader reads the directory back to the original tensors
    import json

    from safetensors.torch import save_file

    directory = tmp_path / 'bundle'
    backbone.save_pretrained(directory / 'backbone', state_dict=state)
    save_file({k: weights['head.' + k].contiguous() for k in checkpoint.HEAD_KEYS}, str(directory / 'head.safetensors'))
    (directory / 'config.json').write_text(json.dumps({'format': 'bongard-v1.3', 'head_rank': 256,
                                                       'parameter_dtype': 'bfloat16'}))
    restored, _, _ = checkpoint.read_checkpoint(directory)
    assert all(torch.equal(restored[name], weights[name]) for name, _ in wl.weight_names(wl.TINY))
