"""Op-level timings of the C-ABI kernels on seeded synthetic inputs.

    python -m bongard_b200.microbench attention [--variant global|window] [--sequences 16]
    python -m bongard_b200.microbench mlp [--tokens 32768]
    python -m bongard_b200.microbench linear [--tokens 32768]
    python -m bongard_b200.microbench glue [--tokens 32768]
    python -m bongard_b200.microbench serve [--shape 4b-4b] [--requests 40] [--no-graphs]
    python -m bongard_b200.microbench dropin [--shape 4b-4b] [--requests 32] [--group 8]
    python -m bongard_b200.microbench train [--layers 2] [--train-sequences 8] [--length 4096]

attention: packed encoder self-attention, lengths uniform in 256-4096 (seed 2), 8 query / 4 KV
heads of 256, QK-norm + RoPE applied by the glue kernel first; FLOPs = 4 D Hq (visible pairs).
mlp: tokens x 2560 -> GeGLU(2 x 10240) -> 2560.  linear: the q|k|v and o projections.
Each op is timed with CUDA events over `--iters` launches after `--warmup`; inputs are larger
than L2 or L2 is flushed between launches (--flush).  Prints one JSON object per op.
serve: wall-clock latency of `serving.Predictor.predict` (host token ids in, probabilities out):
short requests one at a time (distinct states of 256-1024 tokens, one question each; median and
p95 after one pass that captures the buckets), and 32 questions on one 2048-token state as one
request against 32 separate requests (the two workloads the reference quotes latencies for,
README.md:185-186, there on other hardware and real requests).
dropin: the Hugging Face backbone with the hot-path modules substituted (`install_b200_inference`)
driven through the reference's packed call sequence (`hf.PackedJudge.forward_packed`, decoder groups
of 8 questions as the reference forms them), against `JudgmentEngine` on the same weights and
requests: questions/s of both and the largest difference between their probabilities.
train: forward + backward of the first encoder layers at the 4B width in train mode, the substituted
modules on one pack against the native Hugging Face modules on the same sequences as a dense batch
(PyTorch autograd, SDPA): time per step and model TFLOP/s of each.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import ops, workload as wl

DEV = 'cuda'


MIN_SECONDS = 0.4      # every timing loops at least this long, so that the 200 ms clock sampler sees it


def timed(fn, iters, warmup, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if flush is None:
        rounds = 0
        while True:
            begin.record()
            for _ in range(iters):
                fn()
            end.record()
            torch.cuda.synchronize()
            total += begin.elapsed_time(end)
            rounds += 1
            if total >= MIN_SECONDS * 1e3 or iters <= 1:
                return total / (rounds * iters)
    for _ in range(iters):
        flush.zero_()
        begin.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += begin.elapsed_time(end)
    return total / iters


def randn(*shape, std=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * std).bfloat16()


def attention(args, flush):
    lengths = wl.varlen_lengths(2, args.sequences)
    t, hq, hkv, d = sum(lengths), 8, 4, 256
    window, theta = (None, 1e6) if args.variant == 'global' else (1024, 1e4)
    qkv = randn(t, (hq + 2 * hkv) * d, seed=2)
    q = qkv[:, :hq * d].view(t, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(t, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(t, hkv, d)
    gain = torch.zeros(d, device=DEV, dtype=torch.bfloat16)
    positions = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]).to(DEV)
    ops.qk_norm_rope_(q, k, gain, gain, positions, ops.inv_freq(d, theta, DEV))
    plan = ops.make_plan(lengths, window, DEV, group=hq // hkv, head_dim=d, backward=args.backward,
                         pair=False if args.no_pair else (True if args.all_pair else None))
    ms = timed(lambda: ops.varlen_attention(q, k, v, plan, d ** -0.5), args.iters, args.warmup, flush)
    flops = 4 * d * hq * plan.pairs
    out = [dict(op=f'varlen_attention_{args.variant}', tokens=t, sequences=len(lengths), tiles=plan.n_tiles,
                pair_tiles=plan.n_pair_tiles,
                ms=ms, tflops=flops / ms / 1e9, algorithmic_tflop=flops / 1e12,
                min_bytes=2 * t * (2 * hq + 2 * hkv) * d)]
    if args.backward:
        # five contractions per visible pair (S, dP, dV, dK, dQ) against the forward's two
        o, lse = ops.varlen_attention(q, k, v, plan, d ** -0.5, return_lse=True)
        dout = randn(t, hq, d, seed=3)
        ms = timed(lambda: ops.varlen_attention_backward(q, k, v, plan, d ** -0.5, o, lse, dout), args.iters,
                   args.warmup, flush)
        out.append(dict(op=f'varlen_attention_backward_{args.variant}', tokens=t, key_tiles=plan.n_kv_tiles, ms=ms,
                        tflops=2.5 * flops / ms / 1e9, algorithmic_tflop=2.5 * flops / 1e12))
    return out


def mlp(args, flush):
    t, h, i = args.tokens, 2560, 10240
    x = randn(t, h, seed=3)
    wgu, wd = randn(2 * i, h, std=0.02, seed=4), randn(h, i, std=0.02, seed=5)
    out = []
    hidden = ops.linear_geglu(x, wgu)
    for name, fn, flops, nbytes in (
            ('gate_up_geglu', lambda: ops.linear_geglu(x, wgu, few_rows=args.few_rows), 4 * t * h * i, 2 * (t * h + 2 * i * h + t * i)),
            ('down', lambda: ops.linear(hidden, wd, few_rows=args.few_rows), 2 * t * h * i, 2 * (t * i + i * h + t * h))):
        ms = timed(fn, args.iters, args.warmup, flush)
        out.append(dict(op=f'gemm_bf16_{name}', tokens=t, ms=ms, tflops=flops / ms / 1e9, min_bytes=nbytes))
    both = timed(lambda: ops.linear(ops.linear_geglu(x, wgu), wd), args.iters, args.warmup, flush)
    out.append(dict(op='geglu_mlp', tokens=t, ms=both, tflops=6 * t * h * i / both / 1e9))
    if args.fp8:
        qgu, qd = ops.quantize_weight(wgu), ops.quantize_weight(wd)
        xq, xs = ops.quantize_rows(x)
        hq, hs = ops.quantize_rows(hidden)
        for name, fn, flops in (
                ('quantize_rows_x', lambda: ops.quantize_rows(x), 0),
                ('gemm_fp8_gate_up_geglu', lambda: ops.gemm_fp8(xq, xs, qgu, geglu=True), 4 * t * h * i),
                ('gemm_fp8_down', lambda: ops.gemm_fp8(hq, hs, qd), 2 * t * h * i),
                ('geglu_mlp_fp8_with_quantisation',
                 lambda: ops.linear_fp8(ops.linear_fp8(x, qgu, geglu=True), qd), 6 * t * h * i)):
            ms = timed(fn, args.iters, args.warmup, flush)
            out.append(dict(op=name, tokens=t, ms=ms, tflops=flops / ms / 1e9))
        mgu, md = ops.quantize_mxfp8(wgu), ops.quantize_mxfp8(wd)
        xm, hm = ops.quantize_mxfp8(x), ops.quantize_mxfp8(hidden)
        for name, fn, flops in (
                ('quantize_mxfp8_x', lambda: ops.quantize_mxfp8(x), 0),
                ('gemm_mxfp8_gate_up_geglu', lambda: ops.gemm_mxfp8(xm, mgu, geglu=True), 4 * t * h * i),
                ('gemm_mxfp8_down', lambda: ops.gemm_mxfp8(hm, md), 2 * t * h * i),
                ('geglu_mlp_mxfp8_with_quantisation',
                 lambda: ops.linear_mxfp8(ops.linear_mxfp8(x, mgu, geglu=True), md), 6 * t * h * i)):
            ms = timed(fn, args.iters, args.warmup, flush)
            out.append(dict(op=name, tokens=t, ms=ms, tflops=flops / ms / 1e9))
    return out


def linear(args, flush):
    t = args.tokens
    out = []
    for name, n, k in (('qkv', 4096, 2560), ('o', 2560, 2048)):
        x, w = randn(t, k, seed=6), randn(n, k, std=0.02, seed=7)
        ms = timed(lambda: ops.linear(x, w, few_rows=args.few_rows), args.iters, args.warmup, flush)
        out.append(dict(op=f'gemm_bf16_{name}', tokens=t, ms=ms, tflops=2 * t * n * k / ms / 1e9,
                        min_bytes=2 * (t * k + n * k + t * n)))
        if name == 'qkv':
            # the same projection with QK-norm + RoPE in its epilogue, against projection + separate kernel
            gain = randn(256, std=0.1, seed=12)
            positions = (torch.arange(t, device=DEV, dtype=torch.int32) % 4096)
            table = ops.rope_table(256, 1e4, 4096, DEV)
            ms = timed(lambda: ops.linear_qkv_rope(x, w, 2048, 1024, 256, gain, gain, positions, table), args.iters,
                       args.warmup, flush)
            out.append(dict(op='gemm_bf16_qkv_fused_norm_rope', tokens=t, ms=ms, tflops=2 * t * n * k / ms / 1e9))
            freqs = ops.inv_freq(256, 1e4, DEV)

            def two_kernels():
                y = ops.linear(x, w)
                ops.qk_norm_rope_(y[:, :2048].view(t, 8, 256), y[:, 2048:3072].view(t, 4, 256), gain, gain, positions, freqs)

            ms = timed(two_kernels, args.iters, args.warmup, flush)
            out.append(dict(op='gemm_bf16_qkv_then_norm_rope', tokens=t, ms=ms, tflops=2 * t * n * k / ms / 1e9))
        # the weight gradient dW = dy^T x: operands read in place (MN-major tiles) against transposed copies first
        dy = randn(t, n, seed=16)
        ms = timed(lambda: ops.linear_tn(dy, x), args.iters, args.warmup, flush)
        out.append(dict(op=f'gemm_bf16_tn_{name}_weight_gradient', tokens=t, ms=ms, tflops=2 * t * n * k / ms / 1e9))
        ms = timed(lambda: ops.linear(ops.transpose(dy), ops.transpose(x)), args.iters, args.warmup, flush)
        out.append(dict(op=f'gemm_bf16_{name}_weight_gradient_via_transposes', tokens=t, ms=ms,
                        tflops=2 * t * n * k / ms / 1e9))
    return out


def glue(args, flush):
    t, h = args.tokens, 2560
    x, y, w = randn(t, h, seed=8), randn(t, h, seed=9), randn(h, std=0.1, seed=10)
    out = []
    ms = timed(lambda: ops.rmsnorm(x, w), args.iters, args.warmup, flush)
    out.append(dict(op='rmsnorm', tokens=t, ms=ms, gbs=2 * t * h * 2 / ms / 1e6))
    ms = timed(lambda: ops.add_rmsnorm_(y, w, x, w), args.iters, args.warmup, flush)
    out.append(dict(op='add_rmsnorm', tokens=t, ms=ms, gbs=4 * t * h * 2 / ms / 1e6))
    # the fp32 residual stream: fp32 x read by the norm; y and resid fp32 in the update (the engine's default)
    x32, y32 = x.float(), y.float()
    ms = timed(lambda: ops.rmsnorm(x32, w), args.iters, args.warmup, flush)
    out.append(dict(op='rmsnorm_fp32_input', tokens=t, ms=ms, gbs=t * h * (4 + 2) / ms / 1e6))
    ms = timed(lambda: ops.add_rmsnorm_(y, w, x32, w), args.iters, args.warmup, flush)
    out.append(dict(op='add_rmsnorm_fp32_residual', tokens=t, ms=ms, gbs=t * h * (2 + 4 + 4 + 2) / ms / 1e6))
    ms = timed(lambda: ops.add_rmsnorm_(y32, w, x32, w), args.iters, args.warmup, flush)
    out.append(dict(op='add_rmsnorm_fp32_residual_fp32_y', tokens=t, ms=ms, gbs=t * h * (4 + 4 + 4 + 2) / ms / 1e6))
    qkv = randn(t, 4096, seed=11)
    q, k = qkv[:, :2048].view(t, 8, 256), qkv[:, 2048:3072].view(t, 4, 256)
    gain = randn(256, std=0.1, seed=12)
    positions = (torch.arange(t, device=DEV, dtype=torch.int32) % 4096)
    freqs = ops.inv_freq(256, 1e4, DEV)
    ms = timed(lambda: ops.qk_norm_rope_(q, k, gain, gain, positions, freqs), args.iters, args.warmup, flush)
    out.append(dict(op='qk_norm_rope', tokens=t, ms=ms, gbs=2 * t * 3072 * 2 / ms / 1e6))
    table = ops.rope_table(256, 1e4, 4096, DEV)
    ms = timed(lambda: ops.qk_norm_rope_(q, k, gain, gain, positions, None, table=table), args.iters, args.warmup, flush)
    out.append(dict(op='qk_norm_rope_angle_table', tokens=t, ms=ms, gbs=2 * t * 3072 * 2 / ms / 1e6))
    # backward of the two norms: input + upstream gradient in, input gradient out
    ms = timed(lambda: ops.rmsnorm_backward(x, w, y), args.iters, args.warmup, flush)
    out.append(dict(op='rmsnorm_backward', tokens=t, ms=ms, gbs=3 * t * h * 2 / ms / 1e6))
    xq, xk = q.contiguous(), k.contiguous()
    dq, dk = randn(t, 8, 256, seed=13), randn(t, 4, 256, seed=14)
    ms = timed(lambda: ops.qk_norm_rope_backward(xq, xk, gain, gain, dq, dk, positions=positions, freqs=freqs),
               args.iters, args.warmup, flush)
    out.append(dict(op='qk_norm_rope_backward', tokens=t, ms=ms, gbs=3 * t * 3072 * 2 / ms / 1e6))
    return out


def serve(args, flush):
    import statistics
    import time

    from .engine import JudgmentEngine
    from .serving import Predictor

    shape = wl.SHAPES[args.shape]
    ops.SPLIT_K = not args.no_split_k
    engine = JudgmentEngine(wl.make_weights_device(shape, 4, DEV), shape)
    served = Predictor(engine, graphs=not args.no_graphs, programmatic_launch=not args.no_pdl)

    def clock(request):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        served.predict(request)
        return (time.perf_counter() - t0) * 1e3

    short = wl.judged_requests(21, vocab=shape.vocab, requests=args.requests, state=(256, 1024), questions=(1, 1))
    for r in short:
        served.predict(r)                          # captures every bucket these requests touch
    served.clear_state_cache()
    cold = sorted(clock(r) for r in short)          # encoder + projection + decoder per request
    warm = sorted(clock(r) for r in short)          # encoder state cached
    out = [dict(op='serve_short', shape=shape.name, graphs=not args.no_graphs, requests=len(short),
                state_tokens='256-1024', questions=1,
                median_ms=statistics.median(cold), p95_ms=cold[int(0.95 * (len(cold) - 1))],
                cached_state_median_ms=statistics.median(warm), cache=served.state_cache_info())]

    shared = wl.judged_requests(22, vocab=shape.vocab, requests=1, state=(2048, 2048), questions=(32, 32))[0]
    singles = [wl.Request(shared.state, {qid: q}) for qid, q in shared.questions.items()]
    served.predict(shared)
    for r in singles:
        served.predict(r)
    served.clear_state_cache()
    together = min(clock(shared) for _ in range(3) if served.clear_state_cache() is None)
    served.clear_state_cache()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for r in singles:
        served.predict(r)
    separate = (time.perf_counter() - t0) * 1e3
    out.append(dict(op='serve_shared_state', shape=shape.name, graphs=not args.no_graphs, state_tokens=2048, questions=32,
                    one_request_ms=together, separate_requests_ms=separate,
                    question_tokens=sum(len(q.tokens) for q in shared.questions.values())))
    return out


def dropin(args, flush):
    import time

    from transformers import T5Gemma2Model

    from . import install
    from .engine import JudgmentEngine
    from .hf import PackedJudge, hf_config

    shape = wl.SHAPES[args.shape]
    torch.manual_seed(7)
    with torch.device(DEV):
        backbone = T5Gemma2Model(hf_config(shape)).to(torch.bfloat16).eval()
    weights = {k: v for k, v in backbone.state_dict().items()}
    g = torch.Generator(device=DEV).manual_seed(8)
    for name, dims in wl.weight_names(shape):
        if name.startswith('head.'):
            weights[name] = (torch.randn(dims, device=DEV, generator=g) * 0.02).bfloat16()
    requests = wl.judged_requests(23, vocab=shape.vocab, requests=args.requests)
    questions = sum(len(r.questions) for r in requests)
    engine = JudgmentEngine(weights, shape)
    counts = install.install_b200_inference(backbone)
    judge = PackedJudge(backbone, weights)

    def clock(fn):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = fn()
        torch.cuda.synchronize()
        return out, time.perf_counter() - t0

    packed, t_dropin = clock(lambda: judge.forward_packed(requests, args.group))
    probs_engine, t_engine = clock(lambda: engine.judge(requests))
    a = torch.cat([torch.softmax(v['logits'].double(), 0).cpu() for r in packed for v in r.values()])
    b = torch.cat([p for r in probs_engine for p in r.values()])
    # rounding floor of the model itself: the same engine with another summation order in one GEMM per layer
    engine.fuse_qkv_rope = True
    c = torch.cat([p for r in engine.judge(requests) for p in r.values()])
    engine.fuse_qkv_rope = False
    return dict(op='dropin_vs_engine', shape=shape.name, questions_per_decoder_call=args.group, requests=len(requests), questions=questions,
                substituted=counts, dropin_questions_per_s=questions / t_dropin, engine_questions_per_s=questions / t_engine,
                max_abs_prob_diff=float((a - b).abs().max()), mean_abs_prob_diff=float((a - b).abs().mean()),
                floor_max_abs_prob_diff=float((c - b).abs().max()), floor_mean_abs_prob_diff=float((c - b).abs().mean()))


def train(args, flush):
    import dataclasses

    from transformers import T5Gemma2Model

    from . import install, packing
    from .hf import hf_config

    full = wl.SHAPES['4b-4b']
    shape = dataclasses.replace(full, layers=args.layers, layer_types=full.layer_types[:args.layers])
    n, length = args.train_sequences, args.length
    t = n * length
    torch.manual_seed(9)
    with torch.device(DEV):
        backbone = T5Gemma2Model(hf_config(shape)).to(torch.bfloat16).train()
    ids = torch.randint(2, shape.vocab, (n, length), device=DEV)
    dy = randn(n, length, shape.hidden, seed=15)

    # model FLOPs of one step: 2 per multiply-add, forward + 2x backward for the linears; attention forward
    # 4 D Hq pairs, backward 2.5x that (five contractions against two)
    per_token = 2 * (shape.hidden * (shape.q_dim + 2 * shape.kv_dim) + shape.q_dim * shape.hidden
                     + 3 * shape.hidden * shape.intermediate)
    flops = 0.0
    for index in range(shape.layers):
        window = shape.layer_window(index)
        pairs = n * (length * length if window is None else
                     sum(min(length, i + window // 2 + 1) - max(0, i - (window + 1) // 2 + 1) for i in range(length)))
        flops += 3 * per_token * t + 3.5 * 4 * shape.head_dim * shape.q_heads * pairs

    def step_native():
        backbone.zero_grad(set_to_none=True)
        out = backbone.encoder(input_ids=ids, use_cache=False).last_hidden_state
        out.backward(dy)

    ms_native = timed(step_native, args.iters, args.warmup, flush)
    counts = install.install_b200_inference(backbone)
    layout = packing.packed_layout([length] * n, [], DEV)
    empty = torch.empty(0, device=DEV)
    flat_ids, flat_dy = ids.reshape(1, t), dy.reshape(1, t, shape.hidden)

    def step_ours():
        backbone.zero_grad(set_to_none=True)
        out = backbone.encoder(input_ids=flat_ids, position_ids=layout.positions,
                               attention_mask={'full_attention': empty, 'sliding_attention': empty},
                               packed_layout=layout, use_cache=False).last_hidden_state
        out.backward(flat_dy)

    ms_ours = timed(step_ours, args.iters, args.warmup, flush)
    ops.SPLIT_K = False          # the same step without K slices in the small weight-gradient GEMMs
    ms_unsplit = timed(step_ours, args.iters, args.warmup, flush)
    ops.SPLIT_K = True
    ops.GEGLU_KEEP_PREACTIVATIONS = False   # fused GEMM + GeGLU forward, pre-activations recomputed in the backward
    ms_recompute = timed(step_ours, args.iters, args.warmup, flush)
    ops.GEGLU_KEEP_PREACTIVATIONS = True
    return dict(op='encoder_layers_forward_backward', layers=shape.layers, layer_types=list(shape.layer_types),
                sequences=n, length=length, substituted=counts, model_tflop=flops / 1e12,
                native_ms=ms_native, native_tflops=flops / ms_native / 1e9,
                substituted_ms=ms_ours, substituted_tflops=flops / ms_ours / 1e9, substituted_without_k_slices_ms=ms_unsplit,
                substituted_recomputing_geglu_ms=ms_recompute)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('op', choices=['attention', 'mlp', 'linear', 'glue', 'serve', 'dropin', 'train'])
    ap.add_argument('--shape', default='4b-4b', choices=sorted(wl.SHAPES))
    ap.add_argument('--requests', type=int, default=40)
    ap.add_argument('--no-split-k', action='store_true', help='serve: no K slices for under-filled projections')
    ap.add_argument('--layers', type=int, default=2, help='train: encoder layers')
    ap.add_argument('--train-sequences', type=int, default=8, help='train: sequences per step')
    ap.add_argument('--length', type=int, default=4096, help='train: tokens per sequence')
    ap.add_argument('--group', type=int, default=8, help='dropin: questions per decoder call (the reference\'s branch batch size)')
    ap.add_argument('--backward', action='store_true', help='attention: also time the backward passes')
    ap.add_argument('--few-rows', action='store_true', help='linear/mlp: allow the split-K kernel for <= 256 tokens')
    ap.add_argument('--no-pdl', action='store_true', help='serve: plain launches instead of programmatic dependent launch')
    ap.add_argument('--no-graphs', action='store_true', help='serve: launch every kernel eagerly')
    ap.add_argument('--variant', default='global', choices=['global', 'window'])
    ap.add_argument('--sequences', type=int, default=16)
    ap.add_argument('--tokens', type=int, default=32768)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--fp8', action='store_true', help='mlp: also time the E4M3 block-scaled path')
    ap.add_argument('--flush', action='store_true', help='write a 256 MB buffer between launches')
    ap.add_argument('--no-pair', action='store_true', help='attention: 128-row tiles on single CTAs instead of CTA pairs')
    ap.add_argument('--all-pair', action='store_true', help='attention: every run on CTA pairs, also the short rests')
    args = ap.parse_args()
    ops.device_check()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV) if args.flush else None
    from .clocks import ClockSampler

    sampler = ClockSampler(torch.cuda.current_device()).start()
    result = {'attention': attention, 'mlp': mlp, 'linear': linear, 'glue': glue, 'serve': serve, 'dropin': dropin, 'train': train}[args.op](args, flush)
    ops.read_status()
    clocks = sampler.stop()       # SM clock and throttle reasons while the ops above ran: a timing without it proves nothing
    for row in result if isinstance(result, list) else [result]:
        print(json.dumps({**row, 'clocks': clocks}))


if __name__ == '__main__':
    main()
