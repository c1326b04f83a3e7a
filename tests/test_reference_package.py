"""The reference package under oracle/_ref/ is the reference: run on CPU it reproduces the
committed fixtures (which were generated from a reference checkout), through its own
JudgmentModel in all three execution modes and through its own Predictor.predict.

Skipped when oracle/_ref/ has not been created (python oracle/make_ref.py).
"""

import numpy as np
import pytest
import torch

from bongard_b200 import workload as wl
from oracle import reference_package as rp

pytestmark = pytest.mark.skipif(not rp.available(), reason='oracle/_ref is absent: run python oracle/make_ref.py')


def _probs(ref, result):
    return np.concatenate([ref.probabilities(v['logits'].float(), 1.0).numpy() for a in result for v in a.values()])


@torch.inference_mode()
def test_reference_on_cpu_reproduces_the_fixtures(golden_dir):
    ref = rp.load()
    gold = np.load(golden_dir / 'tiny_config1.npz')
    requests = wl.tiny_requests(1)
    compiler = rp.StubCompiler()
    model = rp.build_model(ref, wl.TINY, wl.make_weights(wl.TINY, 1), torch.float32, compiler=compiler)
    ref_requests = rp.to_reference_requests(ref, requests)
    serving = [model(r) for r in ref_requests]
    assert np.abs(_probs(ref, serving) - gold['probs_serving_fp32']).max() < 1e-6
    padded = model(ref_requests)
    assert np.abs(_probs(ref, padded) - gold['probs_serving_fp32']).max() < 1e-5
    model.packing, model.packing_attention = True, 'triton'
    packed = model(ref_requests)
    assert np.abs(_probs(ref, packed) - gold['probs_packed_fp32']).max() < 1e-6
    # the public call: Predictor.predict on the wire form, answers as typed probabilities
    model.packing = False
    predictor = ref.Predictor(model, model_id='tiny')
    got = []
    for i, (request, compiled) in enumerate(zip(requests, ref_requests)):
        compiler.register(f's{i}', compiled)
        reply = predictor.predict(rp.request_json(f's{i}', request))
        assert reply['model'] == 'tiny' and reply['usage']['output_tokens'] == 0
        for qid, q in request.questions.items():
            got.extend(reply['answers'][qid]['probabilities'][key] for key in q.keys)
    assert np.abs(np.asarray(got) - gold['probs_serving_fp32']).max() < 1e-6
