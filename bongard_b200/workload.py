"""Model shapes, seeded random-init weights and seeded synthetic requests.

No checkpoint, tokenizer or benchmark dataset is available offline, so every
measurement and parity case runs on random-init weights and synthetic token
ids whose shapes, lengths and value ranges follow the configurations quoted
for the reference's headline metric.  Lengths come from ``random.Random(seed)``
and values from ``numpy.random.Generator(PCG64(seed))``; both are stable across
machines, so a fixture generated next to the reference can be regenerated on a
GPU host that does not have it.

``Question`` and ``Request`` restate the output contract of the reference's
request compiler (bongard/compiler.py:29-49): the hot path consumes only these.
"""

from __future__ import annotations

import math
import random
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass(frozen=True)
class Question:
    keys: tuple
    tokens: tuple
    candidate_positions: tuple
    decision_position: int
    instruction_tokens: int = 0
    candidate_starts: tuple = ()


@dataclass(frozen=True)
class Request:
    state: tuple
    questions: dict
    input_tokens: int = 0
    images: tuple = ()
    pixel_values: object = field(default=None, compare=False, repr=False)

    @property
    def state_key(self):
        return self.state, self.images


@dataclass(frozen=True)
class ModelShape:
    """Text-stack hyper-parameters of a T5Gemma2-style judgment model."""

    name: str
    vocab: int
    hidden: int
    intermediate: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    window: int
    layer_types: tuple  # 'sliding_attention' | 'full_attention' per layer
    theta_local: float
    theta_global: float
    query_pre_attn_scalar: int
    eps: float = 1e-6
    eoi_token: int = 256_000
    head_rank: int = 256

    @property
    def scale(self):
        return self.query_pre_attn_scalar ** -0.5

    @property
    def q_dim(self):
        return self.q_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.kv_heads * self.head_dim

    def layer_window(self, index):
        return self.window if self.layer_types[index] == 'sliding_attention' else None

    def layer_theta(self, index):
        return self.theta_local if self.layer_types[index] == 'sliding_attention' else self.theta_global

    @property
    def params_per_layer(self):
        h = self.hidden
        return h * (2 * self.q_dim + 2 * self.kv_dim) + 3 * h * self.intermediate


def _pattern(layers):
    # transformers' default: every sixth layer is global ((i + 1) % 6 == 0).
    return tuple('full_attention' if (i + 1) % 6 == 0 else 'sliding_attention' for i in range(layers))


TINY = ModelShape(
    name='tiny', vocab=32768, hidden=256, intermediate=1024, layers=2, q_heads=4, kv_heads=2,
    head_dim=64, window=128, layer_types=('sliding_attention', 'full_attention'),
    theta_local=1e4, theta_global=1e4, query_pre_attn_scalar=64,
)

B4 = ModelShape(
    name='4b-4b', vocab=262144, hidden=2560, intermediate=10240, layers=34, q_heads=8, kv_heads=4,
    head_dim=256, window=1024, layer_types=_pattern(34),
    theta_local=1e4, theta_global=1e6, query_pre_attn_scalar=256,
)

# A two-layer cut of the 4B shape: same kernels and tile shapes, small enough for CPU checks.
B4_SLICE = ModelShape(
    name='4b-slice', vocab=4096, hidden=2560, intermediate=10240, layers=2, q_heads=8, kv_heads=4,
    head_dim=256, window=1024, layer_types=('sliding_attention', 'full_attention'),
    theta_local=1e4, theta_global=1e6, query_pre_attn_scalar=256,
)

SHAPES = {s.name: s for s in (TINY, B4, B4_SLICE)}


# --------------------------------------------------------------------------------------
# weights
# --------------------------------------------------------------------------------------

def weight_names(shape: ModelShape):
    """(name, shape) of every tensor the hot path reads, with Hugging Face key names."""
    h, i, d = shape.hidden, shape.intermediate, shape.head_dim
    names = [('encoder.text_model.embed_tokens.weight', (shape.vocab, h)),
             ('encoder.text_model.embed_tokens.eoi_embedding', (h,)),
             ('encoder.text_model.norm.weight', (h,)),
             ('decoder.norm.weight', (h,))]
    for stack in ('encoder.text_model', 'decoder'):
        for layer in range(shape.layers):
            p = f'{stack}.layers.{layer}.'
            names += [
                (p + 'self_attn.q_proj.weight', (shape.q_dim, h)),
                (p + 'self_attn.k_proj.weight', (shape.kv_dim, h)),
                (p + 'self_attn.v_proj.weight', (shape.kv_dim, h)),
                (p + 'self_attn.o_proj.weight', (h, shape.q_dim)),
                (p + 'self_attn.q_norm.weight', (d,)),
                (p + 'self_attn.k_norm.weight', (d,)),
                (p + 'pre_self_attn_layernorm.weight', (h,)),
                (p + 'post_self_attn_layernorm.weight', (h,)),
                (p + 'mlp.gate_proj.weight', (i, h)),
                (p + 'mlp.up_proj.weight', (i, h)),
                (p + 'mlp.down_proj.weight', (h, i)),
                (p + 'pre_feedforward_layernorm.weight', (h,)),
                (p + 'post_feedforward_layernorm.weight', (h,)),
            ]
    names += [('head.w.weight', (1, h)),
              ('head.candidate.weight', (shape.head_rank, h)),
              ('head.global_readout.weight', (shape.head_rank, h))]
    return names


def make_weights(shape: ModelShape, seed: int, *, std=0.02, norm_std=0.0, dtype=torch.float32, portable=True):
    """Seeded random-init weights as CPU tensors keyed by Hugging Face names.

    Matrices ~ N(0, std).  One-dimensional tensors (RMSNorm gains, stored zero-centred,
    and the end-of-image embedding row) ~ N(0, norm_std); norm_std=0 leaves them at the
    library's initial value, i.e. gain 1.  The decoder embedding is tied to the encoder's.
    """
    if not portable:
        # Faster multi-threaded generator for cases checked inside one process (no fixture involved).
        gen = torch.Generator().manual_seed(seed)
        return {name: (torch.randn(dims, generator=gen) * (std if len(dims) >= 2 else norm_std)).to(dtype)
                for name, dims in weight_names(shape)}
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for name, dims in weight_names(shape):
        if len(dims) >= 2:
            value = rng.standard_normal(dims, dtype=np.float32) * np.float32(std)
        elif norm_std:
            value = rng.standard_normal(dims, dtype=np.float32) * np.float32(norm_std)
        else:
            value = np.zeros(dims, dtype=np.float32)
        out[name] = torch.from_numpy(value).to(dtype)
    return out


def make_weights_device(shape: ModelShape, seed: int, device, *, std=0.02, dtype=torch.bfloat16):
    """Random-init weights generated directly on a device (throughput runs; not reproducible
    across devices, and nothing compares them with a fixture)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = {}
    for name, dims in weight_names(shape):
        if len(dims) >= 2:
            t = torch.empty(dims, device=device, dtype=dtype)
            t.normal_(0.0, std, generator=gen)
        else:
            t = torch.zeros(dims, device=device, dtype=dtype)
        out[name] = t
    return out


def make_weights_host(shape: ModelShape, seed: int, *, std=0.02, dtype=torch.bfloat16, threads=None):
    """Random-init weights on the host, generated by a pool of threads (timing runs of a CPU arm
    at the full model size, where one sequential generator would take minutes).  Every chunk of
    rows draws from its own seeded generator, so the result depends on the seed only."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    out, jobs = {}, []
    for index, (name, dims) in enumerate(weight_names(shape)):
        if len(dims) < 2:
            out[name] = torch.zeros(dims, dtype=dtype)
            continue
        out[name] = torch.empty(dims, dtype=dtype)
        rows = max(1, (1 << 24) // dims[1])
        jobs += [(name, index, r0, min(r0 + rows, dims[0])) for r0 in range(0, dims[0], rows)]

    def fill(job):
        name, index, r0, r1 = job
        gen = torch.Generator().manual_seed((seed * 1_000_003 + index) * 4096 + r0 // max(1, r1 - r0))
        block = torch.randn((r1 - r0, out[name].shape[1]), generator=gen)
        out[name][r0:r1].copy_(block.mul_(std))

    with ThreadPoolExecutor(threads or os.cpu_count() or 1) as pool:
        list(pool.map(fill, jobs))
    return out


# --------------------------------------------------------------------------------------
# requests
# --------------------------------------------------------------------------------------

def _ids(rng, count, vocab, avoid):
    ids = rng.integers(2, vocab, size=count, dtype=np.int64)
    if avoid is not None and avoid < vocab:
        ids[ids == avoid] = avoid - 1
    return tuple(int(v) for v in ids)


def tiny_requests(seed=1, *, vocab=32768, requests=4, questions=3, state=(64, 512),
                  instruction=(16, 64), candidates=(2, 5), eoi=None):
    """4 requests x 3 questions with 64-512 state tokens, 16-64 question tokens, 2-5 candidates."""
    lengths = random.Random(seed)
    values = np.random.Generator(np.random.PCG64(seed))
    out = []
    for _ in range(requests):
        s = lengths.randint(*state)
        qs = {}
        for q in range(questions):
            lq = lengths.randint(*instruction)
            k = lengths.randint(*candidates)
            positions = tuple(sorted(lengths.sample(range(1, lq - 1), k)))
            qs[f'q{q}'] = Question(tuple(f'c{j}' for j in range(k)), _ids(values, lq, vocab, eoi),
                                   positions, lq - 1, lq)
        out.append(Request(_ids(values, s, vocab, eoi), qs, s))
    return out


def structured_question(lengths, values, vocab, eoi, instruction=(16, 128), candidates=(2, 10),
                        candidate_tokens=(4, 16)):
    """BOS, instruction, every candidate followed by its end marker, final decision marker:
    the token structure the reference's request compiler emits (bongard/compiler.py:204-235)."""
    instr = lengths.randint(*instruction)
    k = lengths.randint(*candidates)
    spans = [lengths.randint(*candidate_tokens) for _ in range(k)]
    positions, cursor = [], 1 + instr
    for span in spans:
        cursor += span
        positions.append(cursor)
        cursor += 1
    lq = cursor + 1
    return Question(tuple(f'c{j}' for j in range(k)), _ids(values, lq, vocab, eoi),
                    tuple(positions), lq - 1, instr)


def judged_requests(seed=4, *, vocab=262144, requests=256, state=(512, 8192), questions=(1, 24),
                    eoi=256_000, with_ids=True):
    """The data-parallel throughput workload: `requests` states of 512-8192 tokens with 1-24
    structured questions each."""
    lengths = random.Random(seed)
    values = np.random.Generator(np.random.PCG64(seed))
    out = []
    for _ in range(requests):
        s = lengths.randint(*state)
        nq = lengths.randint(*questions)
        qs = {f'q{q}': structured_question(lengths, values, vocab, eoi) for q in range(nq)}
        state_ids = _ids(values, s, vocab, eoi) if with_ids else tuple(range(s))
        out.append(Request(state_ids, qs, s))
    return out


def long_context_requests(seed=5, *, vocab=262144, requests=32, state=32768, questions=64, eoi=256_000):
    """Shared-evidence stress: every request has one long state read by many questions."""
    return judged_requests(seed, vocab=vocab, requests=requests, state=(state, state),
                           questions=(questions, questions), eoi=eoi)


def varlen_lengths(seed=2, count=16, low=256, high=4096):
    rng = random.Random(seed)
    return [rng.randint(low, high) for _ in range(count)]


# --------------------------------------------------------------------------------------
# work accounting (roofline numerators) and the data-parallel partition
# --------------------------------------------------------------------------------------

def encoder_pairs(length, window):
    """Visible (query, key) pairs of one bidirectional segment."""
    if window is None:
        return length * length
    left, right = (window + 1) // 2, window // 2 + 1   # distance d=q-k: 0<=d<left or 0<-d<right
    total = 0
    for q in range(length):
        total += min(q, left - 1) + 1 + min(length - 1 - q, right - 1)
    return total


def decoder_pairs(length, state, window):
    own = 0
    for q in range(length):
        own += min(q + 1, window) if window is not None else q + 1
    return own + length * state


def request_flops(shape: ModelShape, request: Request):
    """Algorithmic FLOPs of one request: projection/MLP GEMMs, attention over visible pairs,
    and the decoder's state K/V projection.  Norms, RoPE, softmax and the head are excluded."""
    s = len(request.state)
    lq = [len(q.tokens) for q in request.questions.values()]
    gemm = 2 * shape.params_per_layer * shape.layers * (s + sum(lq))
    state_kv = 2 * shape.layers * s * shape.hidden * 2 * shape.kv_dim
    attn = 0
    for layer in range(shape.layers):
        w = shape.layer_window(layer)
        attn += encoder_pairs(s, w)
        attn += sum(decoder_pairs(l, s, w) for l in lq)
    attn *= 4 * shape.head_dim * shape.q_heads
    return gemm + state_kv + attn


def fast_request_cost(shape: ModelShape, request: Request):
    """Closed-form cost used for load balancing (no per-token loops)."""
    s = len(request.state)
    lq = [len(q.tokens) for q in request.questions.values()]
    gemm = 2 * shape.params_per_layer * shape.layers * (s + sum(lq))
    n_local = sum(1 for t in shape.layer_types if t == 'sliding_attention')
    n_global = shape.layers - n_local
    enc = n_global * s * s + n_local * s * min(s, shape.window)
    dec = shape.layers * sum(l * (s + l // 2) for l in lq)
    return gemm + 4 * shape.head_dim * shape.q_heads * (enc + dec)


def partition_requests(costs, world):
    """Longest-processing-time-first: each request goes to the least-loaded rank.

    The reference balances its data-parallel shards the same way
    (bongard/training.py:913-928, shard_update).  Deterministic, so every rank can
    compute the whole assignment locally.  Returns one list of request indices per rank.
    """
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0] * world
    shards = [[] for _ in range(world)]
    for index in order:
        rank = min(range(world), key=lambda r: (loads[r], r))
        shards[rank].append(index)
        loads[rank] += costs[index]
    return [sorted(s) for s in shards]


def reassemble_answers(gathered, shards, requests, per_rank):
    """Answers of a partitioned batch back in request order.

    `gathered` is the concatenation over ranks of `per_rank` values each: rank r's buffer starts with the flat
    per-candidate answers of its requests `shards[r]` (in that order, questions in request order), the rest is
    padding.  Returns one flat tensor in the order a single rank would produce for the whole batch."""
    sizes = [sum(len(q.candidate_positions) for q in r.questions.values()) for r in requests]
    parts = [None] * len(requests)
    for rank, shard in enumerate(shards):
        cursor = rank * per_rank
        for index in shard:
            parts[index] = gathered[cursor:cursor + sizes[index]]
            cursor += sizes[index]
        if cursor > (rank + 1) * per_rank:
            raise ValueError(f'rank {rank} holds more answers than its {per_rank}-value buffer')
    if any(p is None for p in parts):
        raise ValueError('the shards do not cover every request')
    return torch.cat(parts) if parts else gathered[:0]


def embed_scale(shape: ModelShape, dtype):
    """sqrt(hidden) rounded to the weight dtype, as the embedding multiplies it
    (transformers modeling_t5gemma2.py:645)."""
    return float(torch.tensor(math.sqrt(shape.hidden)).to(dtype))
