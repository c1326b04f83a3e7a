"""Import the reference package from oracle/_ref/ (test and benchmark infrastructure only).

`load()` puts oracle/_ref on the import path and returns the handful of reference objects the
drop-in tests and the CPU arm of the benchmark need; `available()` says whether the tree is
there (oracle/make_ref.py creates it).  Also here: the stub compiler and the JSON request form
that let the reference's own `Predictor.predict` run on pre-tokenised synthetic requests - the
reference's compiler needs a Gemma tokenizer, which does not exist offline, and
`JudgmentModel` itself only reads `compiler.tokenizer.pad_token_id` (bongard/model.py:163) and
`compiler.eos` (bongard/packing.py:244).
"""

import sys
import types
from pathlib import Path

REF = Path(__file__).resolve().parent / '_ref'


def available():
    return (REF / 'bongard' / '__init__.py').exists()


def load():
    """Namespace of reference symbols; raises ImportError when oracle/_ref is missing."""
    if not available():
        raise ImportError('oracle/_ref/bongard is missing: run python oracle/make_ref.py next to a reference checkout')
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import bongard
    if Path(bongard.__file__).resolve().parent != (REF / 'bongard').resolve():
        raise ImportError(f'another bongard package is already imported from {bongard.__file__}')
    from bongard import packing
    from bongard.compiler import Question, Request
    from bongard.inference import Predictor, probabilities
    from bongard.model import JudgmentModel

    return types.SimpleNamespace(packing=packing, Question=Question, Request=Request, Predictor=Predictor,
                                 probabilities=probabilities, JudgmentModel=JudgmentModel)


class StubCompiler:
    """Stands in for bongard.compiler.Compiler: `compile(request_json)` returns the pre-built
    Request registered under request_json['state']."""

    def __init__(self, pad_token_id=0, eos=1):
        self.tokenizer = types.SimpleNamespace(pad_token_id=pad_token_id)
        self.eos = eos
        self.image_processor = types.SimpleNamespace(to_dict=lambda: {})
        self.compiled = {}

    def register(self, name, request):
        self.compiled[name] = request

    def compile(self, request):
        return self.compiled[request['state']]


def to_reference_requests(ref, requests):
    """bongard_b200.workload requests as the reference's own dataclasses (bongard/compiler.py:29-49)."""
    return [ref.Request(r.state, {qid: ref.Question(q.keys, q.tokens, q.candidate_positions, q.decision_position,
                                                    q.instruction_tokens) for qid, q in r.questions.items()},
                        r.input_tokens) for r in requests]


def request_json(name, request):
    """The wire form of a synthetic request that passes the reference's validation
    (bongard/data.py validate_question): one `choice` question per Question with as many
    criteria as it has candidates."""
    return {'state': name,
            'questions': {qid: {'type': 'choice', 'instructions': 'synthetic',
                                'criteria': {key: None for key in q.keys}}
                          for qid, q in request.questions.items()}}


def build_model(ref, shape, weights, dtype, device='cpu', compiler=None):
    """The reference's JudgmentModel around a Hugging Face T5Gemma2 backbone of `shape`, loaded
    with Hugging Face-named `weights` (bongard/model.py:142-172).  The backbone is constructed in
    `dtype` without the library's own random initialisation (at the 4B shape that would cost
    minutes and twice the memory); every tensor the text path reads comes from `weights`, the
    vision tower's parameters (never run without pixel values) are zeroed."""
    import torch
    from transformers import T5Gemma2Model

    from bongard_b200.hf import hf_config

    try:
        from transformers.initialization import no_init_weights
    except ImportError:
        from transformers.modeling_utils import no_init_weights

    compiler = compiler or StubCompiler()
    previous = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with no_init_weights():
            backbone = T5Gemma2Model(hf_config(shape))
    finally:
        torch.set_default_dtype(previous)
    model = ref.JudgmentModel(backbone, compiler, dtype=dtype).eval()
    state = {}
    for name, value in weights.items():
        if name.startswith('head.'):
            state[name] = value
        else:
            state['backbone.' + name] = value
            if name.startswith('encoder.text_model.embed_tokens.'):
                state['backbone.decoder.embed_tokens.' + name.rsplit('.', 1)[1]] = value
    missing, unexpected = model.load_state_dict(state, strict=False, assign=False)
    if unexpected or any('vision' not in m and 'multi_modal' not in m for m in missing):
        raise ValueError(f'weights do not match the model: missing {missing}, unexpected {unexpected}')
    own = dict(model.named_parameters())
    with torch.no_grad():
        for name in missing:
            if name in own:
                own[name].zero_()
    return model.to(torch.device(device))
