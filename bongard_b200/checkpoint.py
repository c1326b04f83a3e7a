"""Checkpoint directories of the reference, read straight into the engine's weight layout.

A reference checkpoint (`JudgmentModel.save` / `load`, bongard/model.py:540-665) is a directory

    config.json               format 'bongard-v1.3', head_rank 256, parameter_dtype,
                              optional embedding_scales {'encoder': x, 'decoder': y}, ...
    backbone/config.json      the transformers T5Gemma2Config
    backbone/*.safetensors    Hugging Face-named tensors, one file or shards + index json
    head.safetensors          w.weight [1,H], candidate.weight [256,H], global_readout.weight [256,H]
    tokenizer/, adapter/      (not read here: token ids arrive compiled; LoRA checkpoints must
                              be merged first)

`read_checkpoint` maps it to the dict of Hugging Face-named tensors the engine is built from
(text stacks and head only; the vision tower and the multi-modal projector are not on this
path), streaming tensor by tensor to the target device so a 15 GB checkpoint never needs a
second host copy.  `load_engine` adds the stacking the kernels want (q|k|v and gate|up rows in
one matrix - the reference's own `TELinear` stacking, bongard/te_linear.py:47-55 - and, for
`linears='fp8'`, E4M3 weights with their 128x128 tile scales quantised once at load).
`write_checkpoint` writes the same layout, so weights round-trip and tests need no network.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from .workload import ModelShape, weight_names

FORMATS = ('bongard-v1.3',)
HEAD_KEYS = ('w.weight', 'candidate.weight', 'global_readout.weight')
_TIED = {'decoder.embed_tokens.weight': 'encoder.text_model.embed_tokens.weight',
         'decoder.embed_tokens.eoi_embedding': 'encoder.text_model.embed_tokens.eoi_embedding'}


def shape_from_config(config, *, head_rank=256, name='checkpoint'):
    """ModelShape of a T5Gemma2Config dict (backbone/config.json)."""
    text, dec = config['encoder']['text_config'], config['decoder']
    same = ('vocab_size', 'hidden_size', 'intermediate_size', 'num_hidden_layers', 'num_attention_heads',
            'num_key_value_heads', 'head_dim', 'query_pre_attn_scalar', 'sliding_window', 'layer_types', 'rms_norm_eps')
    for key in same:
        if text[key] != dec[key]:
            raise ValueError(f'encoder and decoder disagree on {key}: {text[key]!r} vs {dec[key]!r}')
    for part in (text, dec):
        if part.get('hidden_activation', 'gelu_pytorch_tanh') != 'gelu_pytorch_tanh':
            raise ValueError(f"unsupported activation {part['hidden_activation']!r} (the kernels fuse tanh-GELU)")
        if part.get('attention_bias'):
            raise ValueError('attention projections with bias are not supported')
    rope = text['rope_parameters']
    theta = lambda kind: float(rope[kind]['rope_theta']) if kind in rope else float(rope.get('rope_theta', 1e4))  # noqa: E731
    for kind in ('sliding_attention', 'full_attention'):
        if kind in rope and rope[kind].get('rope_type', 'default') != 'default':
            raise ValueError(f"unsupported rope_type {rope[kind]['rope_type']!r} for {kind}")
    return ModelShape(
        name=name, vocab=text['vocab_size'], hidden=text['hidden_size'], intermediate=text['intermediate_size'],
        layers=text['num_hidden_layers'], q_heads=text['num_attention_heads'], kv_heads=text['num_key_value_heads'],
        head_dim=text['head_dim'], window=text['sliding_window'], layer_types=tuple(text['layer_types']),
        theta_local=theta('sliding_attention'), theta_global=theta('full_attention'),
        query_pre_attn_scalar=text['query_pre_attn_scalar'], eps=text['rms_norm_eps'],
        eoi_token=config.get('eoi_token_index', 256_000), head_rank=head_rank)


def config_from_shape(shape: ModelShape, max_positions=131072):
    """The part of a T5Gemma2Config that the text stacks and `shape_from_config` use."""
    text = dict(
        vocab_size=shape.vocab, hidden_size=shape.hidden, intermediate_size=shape.intermediate,
        num_hidden_layers=shape.layers, num_attention_heads=shape.q_heads, num_key_value_heads=shape.kv_heads,
        head_dim=shape.head_dim, query_pre_attn_scalar=shape.query_pre_attn_scalar, sliding_window=shape.window,
        layer_types=list(shape.layer_types), rms_norm_eps=shape.eps, hidden_activation='gelu_pytorch_tanh',
        attention_bias=False, max_position_embeddings=max_positions,
        rope_parameters={'sliding_attention': {'rope_type': 'default', 'rope_theta': shape.theta_local},
                         'full_attention': {'rope_type': 'default', 'rope_theta': shape.theta_global}})
    return {'model_type': 't5gemma2', 'eoi_token_index': shape.eoi_token, 'tie_word_embeddings': True,
            'encoder': {'model_type': 't5gemma2_encoder', 'text_config': dict(text, model_type='t5gemma2_text')},
            'decoder': dict(text, model_type='t5gemma2_decoder')}


def _tensor_files(directory):
    """{tensor name: file} over a single safetensors file or an index of shards."""
    from safetensors import safe_open

    index = directory / 'model.safetensors.index.json'
    if index.exists():
        return {k: directory / v for k, v in json.loads(index.read_text())['weight_map'].items()}
    files = sorted(directory.glob('*.safetensors'))
    if not files:
        raise FileNotFoundError(f'no safetensors files under {directory}')
    out = {}
    for path in files:
        with safe_open(path, framework='pt') as f:
            for key in f.keys():
                out[key] = path
    return out


def read_checkpoint(directory, *, device='cpu', dtype=torch.bfloat16):
    """(weights, shape, metadata): every tensor `weight_names(shape)` lists, on `device` in `dtype`."""
    from safetensors import safe_open

    directory = Path(directory)
    metadata = json.loads((directory / 'config.json').read_text())
    if metadata.get('format') not in FORMATS or metadata.get('head_rank') != 256:
        raise ValueError('Unsupported model bundle')               # bongard/model.py:594-598
    if metadata.get('lora'):
        raise ValueError('LoRA checkpoints must be merged into the backbone before loading')
    backbone = directory / 'backbone'
    shape = shape_from_config(json.loads((backbone / 'config.json').read_text()), head_rank=metadata['head_rank'],
                              name=directory.name)
    files = _tensor_files(backbone)
    wanted = {name: dims for name, dims in weight_names(shape) if not name.startswith('head.')}
    weights, handles = {}, {}

    def fetch(path, key):
        if path not in handles:
            handles[path] = safe_open(path, framework='pt').__enter__()
        return handles[path].get_tensor(key)

    try:
        alias = {source: tied for tied, source in _TIED.items()}

        def stored_name(name):
            # transformers writes the encoder's text stack as `encoder.*` on disk and maps it to
            # `encoder.text_model.*` in memory; a tied pair may be stored under either name
            options = [name, name.replace('encoder.text_model.', 'encoder.', 1)]
            if name in alias:
                options.append(alias[name])
            return next((o for o in options if o in files), None)

        for name, dims in wanted.items():
            stored = stored_name(name)
            if stored is None:
                raise KeyError(f'checkpoint has no tensor {name!r}')
            t = fetch(files[stored], stored)
            if tuple(t.shape) != tuple(dims):
                raise ValueError(f'{name}: checkpoint has shape {tuple(t.shape)}, the config implies {tuple(dims)}')
            weights[name] = t.to(device=device, dtype=dtype)
        for tied, source in _TIED.items():                        # tied embeddings are usually stored once
            source = stored_name(source)
            if tied in files and source != tied and not torch.equal(fetch(files[tied], tied), fetch(files[source], source)):
                raise ValueError(f'{tied} differs from {source}: untied embeddings are not supported')
    finally:
        for handle in handles.values():
            handle.__exit__(None, None, None)
    with safe_open(directory / 'head.safetensors', framework='pt') as f:
        for key in HEAD_KEYS:
            weights['head.' + key] = f.get_tensor(key).to(device=device, dtype=dtype)
    for name, dims in weight_names(shape):
        if name.startswith('head.') and tuple(weights[name].shape) != tuple(dims):
            raise ValueError(f'{name}: shape {tuple(weights[name].shape)}, expected {tuple(dims)}')
    return weights, shape, metadata


def load_engine(directory, *, device='cuda', linears='bf16', **engine_options):
    """A JudgmentEngine over a checkpoint directory."""
    from .engine import JudgmentEngine

    weights, shape, metadata = read_checkpoint(directory, device=device)
    scales = metadata.get('embedding_scales')
    engine = JudgmentEngine(weights, shape, device, linears=linears, **engine_options)
    if scales is not None:                                        # bongard/model.py:632-637
        engine.embed_scale_enc, engine.embed_scale_dec = float(scales['encoder']), float(scales['decoder'])
    return engine


def write_checkpoint(directory, weights, shape: ModelShape, *, embedding_scales=None, shard_bytes=None):
    """Write `weights` (Hugging Face names, `head.*` for the head) as a checkpoint directory."""
    from safetensors.torch import save_file

    directory = Path(directory)
    backbone = directory / 'backbone'
    backbone.mkdir(parents=True, exist_ok=True)
    body = {k: v.detach().cpu().contiguous() for k, v in weights.items() if not k.startswith('head.')}
    dtype = next(iter(body.values())).dtype
    if shard_bytes is None:
        save_file(body, str(backbone / 'model.safetensors'), metadata={'format': 'pt'})
    else:
        shards, current, size = [], {}, 0
        for key, value in body.items():
            n = value.numel() * value.element_size()
            if current and size + n > shard_bytes:
                shards.append(current)
                current, size = {}, 0
            current[key] = value
            size += n
        shards.append(current)
        weight_map = {}
        for i, shard in enumerate(shards):
            name = f'model-{i + 1:05d}-of-{len(shards):05d}.safetensors'
            save_file(shard, str(backbone / name), metadata={'format': 'pt'})
            weight_map.update({key: name for key in shard})
        (backbone / 'model.safetensors.index.json').write_text(json.dumps({'metadata': {}, 'weight_map': weight_map}))
    (backbone / 'config.json').write_text(json.dumps(config_from_shape(shape), indent=2) + '\n')
    save_file({key: weights['head.' + key].detach().cpu().contiguous() for key in HEAD_KEYS},
              str(directory / 'head.safetensors'))
    manifest = {'format': FORMATS[0], 'head_rank': shape.head_rank, 'parameter_dtype': str(dtype).removeprefix('torch.')}
    if embedding_scales is not None:
        manifest['embedding_scales'] = {'encoder': float(embedding_scales[0]), 'decoder': float(embedding_scales[1])}
    (directory / 'config.json').write_text(json.dumps(manifest, indent=2) + '\n')
    return directory
