"""One switch that substitutes every hot-path module of a T5Gemma2 judgment backbone.

In the reference, kernels are plugged in by in-place module substitution
(`install_shared_attention` bongard/attention.py:286-289, `install_mps_inference`
bongard/mps_inference.py:173-180, `enable_fused_mlp`, `enable_te_linear`, `enable_float8`).
`install_b200_inference` performs the same swaps with the B200 modules: attention modules of
both stacks, every RMSNorm, and the MLPs; the substituted modules reuse the native parameter
objects and accept the keyword arguments the reference threads through the layers.
"""

from __future__ import annotations

from . import ops
from .attention import B200DecoderAttention, B200EncoderAttention, B200RMSNorm
from .te_linear import B200MLP


def install_b200_inference(model, *, linears='bf16'):
    """Swap the hot path of `model` (a JudgmentModel-like object with `.backbone`, or the
    Hugging Face T5Gemma2Model itself) to the B200 kernels.  Returns substitution counts."""
    if linears not in ('bf16', 'fp8', 'mxfp8'):
        raise ValueError("linears must be 'bf16', 'fp8' or 'mxfp8'")
    ops.device_check()
    backbone = model.backbone if hasattr(model, 'backbone') else model
    counts = dict(encoder_attention=0, decoder_attention=0, mlp=0, norms=0)
    for layer in backbone.encoder.text_model.layers:
        if not isinstance(layer.self_attn, B200EncoderAttention):
            layer.self_attn = B200EncoderAttention(layer.self_attn)
        counts['encoder_attention'] += 1
    for layer in backbone.decoder.layers:
        if not isinstance(layer.self_attn, B200DecoderAttention):
            layer.self_attn = B200DecoderAttention(layer.self_attn)
        counts['decoder_attention'] += 1
    for layer in list(backbone.encoder.text_model.layers) + list(backbone.decoder.layers):
        if not isinstance(layer.mlp, B200MLP):
            layer.mlp = B200MLP(layer.mlp, linears)
        counts['mlp'] += 1
    text_roots = [backbone.encoder.text_model, backbone.decoder]
    for root in text_roots:
        for parent in root.modules():
            for name, child in list(parent.named_children()):
                if type(child).__name__.endswith('RMSNorm') and not isinstance(child, B200RMSNorm) \
                        and hasattr(child, 'weight') and hasattr(child, 'eps'):
                    setattr(parent, name, B200RMSNorm(child))
                    counts['norms'] += 1
    if hasattr(model, 'packing_attention'):
        # the reference's forward_packed asks packed_layout for this backend (bongard/packing.py:247-252,
        # 284-289); the name it calls is bound to a dispatcher that serves it, no source is edited
        from .packing import serve_reference_packing

        model.packing_attention = 'b200'
        serve_reference_packing()
    return counts
