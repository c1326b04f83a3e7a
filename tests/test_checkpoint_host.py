"""Checkpoint directories (the reference's save/load layout, bongard/model.py:540-665) round-trip
through the loader on the host: single file and shards, tied embeddings, shape from the
transformers config, and the errors the reference raises for unsupported bundles."""

import json

import pytest
import torch

from bongard_b200 import checkpoint as ck, workload as wl


def test_round_trip_single_file_and_shards(tmp_path):
    weights = wl.make_weights(wl.TINY, 3, norm_std=0.1, dtype=torch.bfloat16)
    for name, shard in (('one', None), ('many', 1 << 20)):
        directory = ck.write_checkpoint(tmp_path / name, weights, wl.TINY, shard_bytes=shard)
        got, shape, meta = ck.read_checkpoint(directory)
        assert shape == ck.shape_from_config(ck.config_from_shape(wl.TINY), name=name)
        assert {f: getattr(shape, f) for f in wl.TINY.__dataclass_fields__ if f != 'name'} == \
               {f: getattr(wl.TINY, f) for f in wl.TINY.__dataclass_fields__ if f != 'name'}
        assert set(got) == {n for n, _ in wl.weight_names(wl.TINY)}
        assert all(torch.equal(got[k], weights[k]) for k in got)
        assert meta['format'] == 'bongard-v1.3' and meta['parameter_dtype'] == 'bfloat16'
    assert len(list((tmp_path / 'many' / 'backbone').glob('model-*.safetensors'))) > 1


def test_reads_a_transformers_saved_backbone(tmp_path):
    """backbone/ written by transformers' own save_pretrained (tied embeddings stored once, vision
    tower present) loads to the same tensors."""
    pytest.importorskip('transformers')
    from safetensors.torch import save_file

    from bongard_b200.hf import build_backbone

    weights = wl.make_weights(wl.TINY, 5, norm_std=0.1)
    backbone = build_backbone(wl.TINY, weights, device='cpu', dtype=torch.float32)
    directory = tmp_path / 'hf'
    backbone.save_pretrained(directory / 'backbone')
    save_file({k: weights['head.' + k].contiguous() for k in ck.HEAD_KEYS}, str(directory / 'head.safetensors'))
    (directory / 'config.json').write_text(json.dumps(
        {'format': 'bongard-v1.3', 'head_rank': 256, 'parameter_dtype': 'float32',
         'embedding_scales': {'encoder': 16.0, 'decoder': 15.5}}))
    got, shape, meta = ck.read_checkpoint(directory, dtype=torch.float32)
    assert (shape.hidden, shape.layers, shape.window, shape.layer_types) == \
           (wl.TINY.hidden, wl.TINY.layers, wl.TINY.window, wl.TINY.layer_types)
    assert (shape.theta_local, shape.theta_global, shape.eoi_token) == (1e4, 1e4, 256_000)
    assert all(torch.equal(got[k], weights[k]) for k in got)
    assert meta['embedding_scales'] == {'encoder': 16.0, 'decoder': 15.5}


def test_rejects_unsupported_bundles(tmp_path):
    weights = wl.make_weights(wl.TINY, 3, dtype=torch.bfloat16)
    directory = ck.write_checkpoint(tmp_path / 'c', weights, wl.TINY)
    manifest = json.loads((directory / 'config.json').read_text())
    (directory / 'config.json').write_text(json.dumps(dict(manifest, format='bongard-v1.2')))
    with pytest.raises(ValueError, match='Unsupported model bundle'):
        ck.read_checkpoint(directory)
    (directory / 'config.json').write_text(json.dumps(dict(manifest, lora={'base': '..'})))
    with pytest.raises(ValueError, match='LoRA'):
        ck.read_checkpoint(directory)
    (directory / 'config.json').write_text(json.dumps(manifest))
    config = json.loads((directory / 'backbone' / 'config.json').read_text())
    config['decoder']['hidden_size'] = 128
    (directory / 'backbone' / 'config.json').write_text(json.dumps(config))
    with pytest.raises(ValueError, match='disagree on hidden_size'):
        ck.read_checkpoint(directory)
    config['decoder']['hidden_size'] = 256
    config['encoder']['text_config']['intermediate_size'] = config['decoder']['intermediate_size'] = 512
    (directory / 'backbone' / 'config.json').write_text(json.dumps(config))
    with pytest.raises(ValueError, match='the config implies'):
        ck.read_checkpoint(directory)
