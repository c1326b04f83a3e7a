"""Single-request serving path: the reference's `Predictor.predict` flow
(bongard/inference.py:283-340 -> bongard/model.py:313-458: `encode` -> `state_kv` ->
`decode_batch` per question group -> head -> probabilities) with its encoder-state LRU
(bongard/inference.py:213-282), built for latency instead of throughput.

What differs from the packed throughput engine:

* One request at a time.  All questions of the request are decoded as ONE packed run over the
  shared state (no padding between questions, no groups of eight): rows are independent, so
  the result equals the grouped form.
* Every stage runs on fixed-size buffers per length bucket, so the ~350 kernel launches of a
  stack are captured once in a CUDA graph and replayed: `encode[Sb]`, `state_kv[Sb]`,
  `decode[Sb, Tb]`.  A bucket pads the token axis with one extra segment of pad tokens
  (owner without a state in the decoder), which keeps every padded row finite and costs no
  attention work beyond that segment; attention plans are padded with empty tiles.
* The state cache holds encoder hidden states (as the reference does) under a byte limit with
  LRU eviction; the bucket also remembers which state its projected K/V currently hold, so
  consecutive requests on one state skip both the encoder and the K/V projection.
* Stacks of up to 256 tokens (a question group against a cached state) run their projections
  on the split-K weight-streaming GEMM (`bg_gemm_bf16_skinny`), which is bound by HBM bandwidth
  instead of by the 10-20 CTAs a 256-wide output tiling would give them.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib, ops
from .engine import DevicePack, JudgmentEngine

BF16 = torch.bfloat16


class StateCache:
    """LRU of encoder states by bytes (bongard/inference.py:229-282: `_cached_state`,
    `_retain_state`, `state_cache_info`, `clear_state_cache`)."""

    def __init__(self, limit_bytes):
        self.limit = int(limit_bytes)
        self.entries = OrderedDict()
        self.bytes = self.hits = self.misses = 0

    @staticmethod
    def size_of(key, state):
        # retained tensor + key payload (bongard/inference.py:224-227)
        tokens, images = key
        return state.numel() * state.element_size() + 36 * len(tokens) + sum(map(len, images))

    def get(self, key):
        if key in self.entries:
            self.hits += 1
            self.entries.move_to_end(key)
            return self.entries[key]
        self.misses += 1
        return None

    def put(self, key, state):
        if not self.limit or key in self.entries:
            return
        size = self.size_of(key, state)
        if size > self.limit:
            return
        while self.bytes + size > self.limit:
            old_key, old = self.entries.popitem(last=False)
            self.bytes -= self.size_of(old_key, old)
        self.entries[key] = state
        self.bytes += size

    def clear(self):
        self.entries.clear()
        self.bytes = 0

    def info(self):
        return {'entries': len(self.entries), 'bytes': self.bytes, 'limit_bytes': self.limit,
                'hits': self.hits, 'misses': self.misses}


def _round_up(n, step):
    return (n + step - 1) // step * step


def _bucket(n, step, fine=32, fine_up_to=256):
    """Bucket size for n tokens: multiples of `step`, but of `fine` up to `fine_up_to` tokens, where
    the few-row GEMM's cost follows the row count and padding 130 tokens to 256 would double it."""
    n = max(int(n), 1)
    return _round_up(n, min(step, fine)) if n <= fine_up_to else _round_up(n, step)


@dataclass
class _Inputs:
    """Fixed-size device inputs of one stack with their pinned host mirror."""

    tokens: int
    host_ids: torch.Tensor
    host_ints: torch.Tensor
    ids: torch.Tensor
    ints: torch.Tensor
    pack: DevicePack
    offsets: dict           # window -> offset of its plan inside ints
    plan_tiles: int
    tail: int = 0           # offset of the free-form tail (readout rows, question offsets)
    copied: object = None   # event after the last host-to-device copies of the mirror


class _Stage:
    """One captured (or eager) stage: run() replays the graph or calls the function."""

    def __init__(self, body, use_graph, engine):
        def fn():
            # latency settings: the few-row GEMM for small stacks, and launches that let a kernel's prologue
            # overlap its predecessor's tail (captured into the graph as programmatic edges)
            previous, engine.few_rows_kernels = engine.few_rows_kernels, True
            lib = _lib.load()
            lib.bg_set_programmatic_launch(1 if engine.programmatic_launch else 0)
            try:
                return body()
            finally:
                engine.few_rows_kernels = previous
                lib.bg_set_programmatic_launch(0)

        self.fn, self.graph, self.out = fn, None, None
        self.out = fn()                       # eager warm-up: lazy library init, allocator warm
        if use_graph:
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, capture_error_mode='thread_local'):
                self.out = fn()

    def run(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.out = self.fn()
        return self.out


class Predictor:
    """`predict(request)` for one `workload.Request`: {question id: float64 probabilities}."""

    def __init__(self, engine: JudgmentEngine, *, state_cache_mib=1024, graphs=True, state_bucket=256,
                 question_bucket=128, fine_bucket=32, max_graph_state=16384, max_graph_question=8192,
                 programmatic_launch=True):
        self.engine, self.graphs = engine, bool(graphs)
        engine.programmatic_launch = bool(programmatic_launch)
        self.cache = StateCache(int(state_cache_mib) * 2 ** 20)
        self.state_bucket, self.question_bucket = int(state_bucket), int(question_bucket)
        self.fine_bucket = int(fine_bucket)   # granularity up to 256 tokens (see _bucket)
        self.max_graph_state, self.max_graph_question = int(max_graph_state), int(max_graph_question)
        s = engine.shape
        self.windows = list(dict.fromkeys(s.layer_window(i) for i in range(s.layers)))
        self.keys = [s.layer_window(i) for i in range(s.layers)]
        self.group = s.q_heads // s.kv_heads
        self.tile_tokens = ops.tile_rows(s.head_dim) // self.group
        self._enc, self._kv, self._dec = {}, {}, {}
        self.graph_replays = 0

    # ------------------------------------------------------------------ fixed-size inputs
    def _inputs(self, tokens):
        device = self.engine.device
        plan_tiles = tokens // self.tile_tokens + 2
        plan_ints = plan_tiles * 8 + 2 * tokens
        tail = tokens + len(self.windows) * plan_ints       # readout rows and question offsets ride along
        n_ints = tail + 3 * tokens + 1
        host_ids = torch.zeros(tokens, dtype=torch.int64).pin_memory()
        host_ints = torch.zeros(n_ints, dtype=torch.int32).pin_memory()
        ids, ints = host_ids.to(device), host_ints.to(device)
        offsets, plans = {}, {}
        rows = ops.tile_rows(self.engine.shape.head_dim)
        for i, w in enumerate(self.windows):
            offsets[w] = tokens + i * plan_ints
            plans[w] = ops.HostPlan(np.zeros(plan_ints, dtype=np.int32), tokens, plan_tiles, 0, rows).view(
                ints[offsets[w]:offsets[w] + plan_ints])
        pack = DevicePack(ids, ints[:tokens], self.keys, plans)
        return _Inputs(tokens, host_ids, host_ints, ids, ints, pack, offsets, plan_tiles, tail)

    def _fill(self, inp, sequences, *, state_length=None, tail=None):
        """Write token ids, positions and padded attention plans of `sequences` (+ one pad
        segment up to the bucket size) into the pinned mirror and start the two copies."""
        s = self.engine.shape
        if inp.copied is not None:
            inp.copied.synchronize()          # the mirror is free again once its last copies are done
        lengths = [len(seq) for seq in sequences]
        used = sum(lengths)
        pad = inp.tokens - used
        ids, ints = inp.host_ids.numpy(), inp.host_ints.numpy()
        cursor = 0
        for seq, n in zip(sequences, lengths):
            ids[cursor:cursor + n] = seq
            ints[cursor:cursor + n] = np.arange(n, dtype=np.int32)
            cursor += n
        if pad:
            ids[used:] = 0
            ints[used:inp.tokens] = np.arange(pad, dtype=np.int32)
            lengths = lengths + [pad]
        decoder = state_length is not None
        owners = state_lengths = None
        if decoder:
            owners = [0] * len(sequences) + ([1] if pad else [])
            state_lengths = [state_length, 0]
        for w, offset in inp.offsets.items():
            hp = ops.make_host_plan(lengths, w, group=self.group, owners=owners, state_lengths=state_lengths,
                                    head_dim=s.head_dim, pair=False).padded(inp.tokens, inp.plan_tiles)
            ints[offset:offset + hp.packed.size] = hp.packed
        if tail is not None:
            ints[inp.tail:inp.tail + len(tail)] = tail
        inp.ids.copy_(inp.host_ids, non_blocking=True)
        inp.ints.copy_(inp.host_ints, non_blocking=True)
        inp.copied = torch.cuda.Event()
        inp.copied.record()

    # ------------------------------------------------------------------ stages
    def _use_graph(self, tokens, limit):
        return self.graphs and tokens <= limit

    def _encoder(self, sb):
        if sb not in self._enc:
            e = self.engine
            inp = self._inputs(sb)
            self._fill(inp, [[0] * sb])
            stage = _Stage(lambda: e._stack(e.enc, e.enc_norm, inp.pack), self._use_graph(sb, self.max_graph_state), e)
            self._enc[sb] = (inp, stage)
        return self._enc[sb]

    def _state_kv(self, sb):
        if sb not in self._kv:
            e = self.engine
            state_in = torch.zeros(sb, e.shape.hidden, device=e.device, dtype=BF16)
            stage = _Stage(lambda: e.state_kv(state_in), self._use_graph(sb, self.max_graph_state), e)
            self._kv[sb] = {'state_in': state_in, 'stage': stage, 'holds': None}
        return self._kv[sb]

    def _decoder(self, sb, tb):
        if (sb, tb) not in self._dec:
            e = self.engine
            kv = self._state_kv(sb)
            inp = self._inputs(tb)
            self._fill(inp, [[0] * tb], state_length=1)
            # a captured decoder reads the state K/V at fixed addresses, which only a captured
            # projection stage provides
            stage = _Stage(lambda: e._stack(e.dec, e.dec_norm, inp.pack, kv['stage'].out),
                           self._use_graph(tb, self.max_graph_question) and kv['stage'].graph is not None, e)
            self._dec[(sb, tb)] = (inp, stage)
        return self._dec[(sb, tb)]

    def _run(self, stage):
        if stage.graph is not None:
            self.graph_replays += 1
        return stage.run()

    # ------------------------------------------------------------------ the request
    @torch.inference_mode()
    def logits(self, request):
        """(candidate logits fp32 [sum of candidates] on the device in question order, device
        offsets int32 [questions + 1] into them, the same offsets as a host list)."""
        e = self.engine
        n_state = len(request.state)
        sb = _bucket(n_state, self.state_bucket, self.fine_bucket)
        kv = self._state_kv(sb)
        key = request.state_key
        if kv['holds'] != key:
            state = self.cache.get(key)
            if state is None:
                inp, stage = self._encoder(sb)
                self._fill(inp, [request.state])
                hidden = self._run(stage)
                self.cache.put(key, hidden[:n_state].clone())
                kv['state_in'].copy_(hidden)
            else:
                kv['state_in'][:n_state].copy_(state)
            kv['holds'] = None
            self._run(kv['stage'])
            kv['holds'] = key
        else:
            self.cache.get(key)                     # keeps the LRU order and the hit count honest
        questions = list(request.questions.values())
        total = sum(len(q.tokens) for q in questions)
        tb = _bucket(total, self.question_bucket, self.fine_bucket)
        inp, stage = self._decoder(sb, tb)
        cand, dec, sizes, offset = [], [], [0], 0
        for q in questions:
            cand.extend(offset + p for p in q.candidate_positions)
            dec.extend([offset + q.decision_position] * len(q.candidate_positions))
            sizes.append(sizes[-1] + len(q.candidate_positions))
            offset += len(q.tokens)
        n = len(cand)
        # readout rows and per-question candidate offsets travel in the same copy as the plans
        self._fill(inp, [q.tokens for q in questions], state_length=n_state, tail=cand + dec + sizes)
        hidden = self._run(stage)
        rows = inp.ints[inp.tail:inp.tail + 2 * n + len(sizes)]
        logits = ops.judgment_head(hidden, rows[:n], rows[n:2 * n], e.head_w, e.head_c, e.head_g)
        return logits, rows[2 * n:], sizes

    @torch.inference_mode()
    def predict(self, request, temperature=1.0):
        """{question id: float64 probabilities [K]} with one device-to-host read
        (bongard/inference.py:305-321)."""
        logits, offsets, sizes = self.logits(request)
        probs = ops.candidate_softmax(logits, offsets, temperature).cpu()
        ops.read_status()
        return {qid: probs[lo:hi] for qid, lo, hi in zip(request.questions, sizes, sizes[1:])}

    def state_cache_info(self):
        return self.cache.info()

    def clear_state_cache(self):
        self.cache.clear()
        for kv in self._kv.values():
            kv['holds'] = None
