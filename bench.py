"""Judged questions per second at the 4B-4B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one pass of the whole hot path (encoder over every state, state K/V projection,
decoder over every question, judgment head, candidate softmax) over one batch of seeded
synthetic requests: 256 requests, states of 512-8192 tokens, 1-24 questions each.  Every rank
holds a full bf16 replica and its own batch (rank r uses seed 4 + r), so the headline scaling is
weak; the only collective is the gather of answers.

`value` times the kernels with the batch already staged in HBM; `e2e` times the public
call JudgmentEngine.judge() from host request objects (host layout, pinned copies, kernels,
one device-to-host copy of the probabilities).  The dominant kernel (the BF16 tensor-core
GEMM) is timed live with CUDA events for the roofline entry.

Extra keys, each timed in the same process with its own clock record:
  strong        (N > 1) ONE seed-4 batch split over the ranks longest-processing-time first;
                answers gathered on rank 0 and compared with rank 0's own run of the whole batch
  long_context  32768-token states x 64 questions, 4 requests per GPU, bf16 / fp8 / mxfp8 linears
  ops           (N = 1) packed encoder attention of 16 sequences (global and window 1024), the
                GeGLU MLP at 32768 tokens in bf16 / fp8 / mxfp8, and the library peaks measured the
                same way in the same run (torch.matmul bf16, torch._scaled_mm e4m3, 8192^3)
  cpu_baseline  (N = 1) the reference's own device="cpu" Predictor on a bounded sample

`--impl reference` times the unmodified reference package (oracle/_ref: bongard.inference
.Predictor.predict on device="cpu") on the host cores; when that tree is absent, the oracle's
restatement of the same path, labelled "port".
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from bongard_b200 import workload as wl  # noqa: E402
from bongard_b200.clocks import ClockSampler  # noqa: E402

METRIC = 'judged_questions_per_second'
UNIT = 'questions/s'
# DRAM bytes per algorithmic FLOP of the bf16 GEMM, measured by ncu on the 8192-token MLP GEMMs
# ((325.9 + 566.8) MB over (0.859 + 0.429) TFLOP); a full-size launch is scaled by its FLOPs.
GEMM_TRAFFIC_PER_FLOP = 6.9e-4


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=2)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--shape', default='4b-4b', choices=sorted(wl.SHAPES))
    ap.add_argument('--requests', type=int, default=256, help='requests per rank per step')
    ap.add_argument('--seed', type=int, default=None, help='default: 4 (judged), 5 (long)')
    ap.add_argument('--workload', default='judged', choices=['judged', 'long'],
                    help="judged: 512-8192-token states, 1-24 questions; long: 32768-token states x 64 questions")
    ap.add_argument('--programmatic-launches', action='store_true',
                    help='launch kernels with programmatic stream serialization')
    ap.add_argument('--linears', default='bf16', choices=['bf16', 'fp8', 'mxfp8'], help='projection / MLP GEMM precision')
    ap.add_argument('--residual', default='fp32wide', choices=['bf16', 'fp32', 'fp32wide'],
                    help='residual stream: fp32 with the output / down projections handed over unrounded (default, the\n'
                         'mode that meets the 1e-3 probability bound), fp32, or bf16 (the reference bf16 chain, 3 %% faster)')
    ap.add_argument('--cpu-seconds', type=float, default=None,
                    help='CPU work per sample (default: 15 s, less when many steps are asked for)')
    ap.add_argument('--encoder-pack-tokens', type=int, default=65536)
    ap.add_argument('--decoder-pack-tokens', type=int, default=32768)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-extras', action='store_true', help='skip the strong / long_context / ops keys')
    ap.add_argument('--extra-steps', type=int, default=2, help='timed steps of the strong and long_context runs')
    args = ap.parse_args()
    if args.seed is None:
        args.seed = 5 if args.workload == 'long' else 4
    if args.workload == 'long' and args.requests == 256:
        args.requests = 4          # four 32768-token states with 64 questions each per GPU
    if args.cpu_seconds is None:
        args.cpu_seconds = 15.0 if args.impl == 'b200' else max(3.0, min(15.0, 240.0 / (args.steps + args.warmup)))
    return args


def peaks():
    path = ROOT / 'MEASURED_PEAKS.json'
    if path.exists():
        data = json.loads(path.read_text())
        return dict(hbm=data['hbm_gbs'], burst=data['bf16_tflops'], sustained=data['bf16_tflops_sustained'], source='measured')
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, source='fallback')


def make_requests(shape, seed, count, workload='judged'):
    if shape.name == 'tiny':
        return wl.tiny_requests(seed, requests=count, questions=3)
    if workload == 'long':
        return wl.long_context_requests(seed, vocab=shape.vocab, requests=count, eoi=shape.eoi_token)
    return wl.judged_requests(seed, vocab=shape.vocab, requests=count, eoi=shape.eoi_token)


def workload_name(shape, args):
    if args.workload == 'judged':
        return (f'{shape.name} judged requests: {args.requests} requests per GPU per step, states 512-8192 tokens, '
                f'1-24 questions each in decoder groups of 8 (seed {args.seed} + rank)')
    return (f'{shape.name} long-context shared evidence: {args.requests} requests per GPU per step, 32768-token '
            f'states, 64 questions each in decoder groups of 8 (seed {args.seed} + rank)')


# --------------------------------------------------------------------------------------
# CPU arm: the reference's own device="cpu" Predictor (oracle/_ref), else the oracle's restatement
# --------------------------------------------------------------------------------------

def cpu_matmul_tflops(dtype):
    a = torch.randn(2048, 2560).to(dtype)
    b = torch.randn(10240, 2560).to(dtype)
    torch.matmul(a, b.t())
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 1.0:
        torch.matmul(a, b.t())
        reps += 1
    return reps * 2 * 2048 * 2560 * 10240 / (time.perf_counter() - t0) / 1e12


def cpu_sample(shape, requests, budget_seconds, efficiency):
    """A bounded sample that looks like the batch: requests whose work per question is closest to
    the batch's average (state tokens per question decide how expensive a judged question is), as
    many as fit a FLOP budget derived from a one-second matmul calibration (`efficiency` = the
    share of the matmul rate the whole path reaches).  Returns (sample, work per question of the
    sample / of the batch)."""
    rate = cpu_matmul_tflops(torch.bfloat16) * 1e12 * efficiency
    budget = rate * budget_seconds
    costs = [wl.fast_request_cost(shape, r) for r in requests]
    counts = [len(r.questions) for r in requests]
    average = sum(costs) / sum(counts)
    order = sorted(range(len(requests)), key=lambda i: (abs(costs[i] / counts[i] / average - 1.0), i))
    chosen, spent = [], 0.0
    for i in order:
        if abs(costs[i] / counts[i] / average - 1.0) > 0.5:
            break
        if spent + costs[i] <= budget:
            chosen.append(requests[i])
            spent += costs[i]
    if not chosen:
        # nothing representative fits: the cheapest request that is still within 50 % of the batch's work
        # per question, however long it takes (one request bounds it); failing that, the cheapest request
        near = [i for i in order if abs(costs[i] / counts[i] / average - 1.0) <= 0.5] or list(range(len(requests)))
        i = min(near, key=lambda j: costs[j])
        chosen, spent = [requests[i]], costs[i]
    ratio = spent / sum(len(r.questions) for r in chosen) / average
    return chosen, ratio


def describe(sample, ratio, how):
    return (f'{len(sample)} request(s) of the step batch chosen for work per question close to the batch average '
            f'({ratio:.2f}x): {sum(len(r.state) for r in sample)} state tokens, {sum(len(r.questions) for r in sample)} '
            f'questions, bf16, {how}, torch CPU with {torch.get_num_threads()} threads')


class CpuArm:
    """One bounded sample of the workload through the reference's CPU path."""

    def __init__(self, shape, weights, requests, budget_seconds):
        from oracle import reference_package as rp

        self.shape = shape
        torch.set_num_threads(os.cpu_count() or 1)
        self.kind = 'reference' if rp.available() else 'port'
        if self.kind == 'reference':
            # the serving path (one request at a time, dense masks, padded decoder batches, fp32 score
            # tiles) reaches about a fifth of the host's bf16 matmul rate
            self.sample, self.ratio = cpu_sample(shape, requests, budget_seconds, 0.2)
            ref = rp.load()
            self.compiler = rp.StubCompiler()
            model = rp.build_model(ref, shape, weights, torch.bfloat16, 'cpu', self.compiler)
            self.predictor = ref.Predictor(model, model_id=shape.name)
            self.wire = []
            for i, (r, compiled) in enumerate(zip(self.sample, rp.to_reference_requests(ref, self.sample))):
                self.compiler.register(f'state-{i}', compiled)
                self.wire.append(rp.request_json(f'state-{i}', r))
            self.how = "the reference's bongard.inference.Predictor.predict on device='cpu' (oracle/_ref)"
        else:
            self.sample, self.ratio = cpu_sample(shape, requests, budget_seconds, 0.5)
            self.weights = weights
            self.how = "oracle restatement of the reference's packed CPU path (oracle/_ref absent)"
        self.questions = sum(len(r.questions) for r in self.sample)

    def step(self):
        """Seconds for one pass over the sample."""
        t0 = time.perf_counter()
        if self.kind == 'reference':
            for request in self.wire:
                reply = self.predictor.predict(request)
                assert len(reply['answers']) == len(request['questions'])
        else:
            from oracle import reference_math as om

            with torch.inference_mode():
                for answers in om.forward_packed(self.weights, self.shape, self.sample, 8, dtype=torch.bfloat16):
                    for v in answers.values():
                        om.probabilities(v['logits'].float())
        return time.perf_counter() - t0

    def describe(self):
        return describe(self.sample, self.ratio, self.how)


def dist_setup():
    return int(os.environ.get('WORLD_SIZE', '1')), int(os.environ.get('RANK', '0')), int(os.environ.get('LOCAL_RANK', '0'))


def run_reference(args):
    """The reference's CPU path on the host cores; rank 0 only, the other ranks leave at once."""
    world, rank, _ = dist_setup()
    if rank != 0:
        return
    shape = wl.SHAPES[args.shape]
    torch.set_num_threads(os.cpu_count() or 1)
    weights = wl.make_weights_host(shape, args.seed)
    requests = make_requests(shape, args.seed, args.requests, args.workload)
    arm = CpuArm(shape, weights, requests, args.cpu_seconds)
    del weights
    for _ in range(args.warmup):
        arm.step()
    elapsed = sum(arm.step() for _ in range(args.steps))
    value = arm.questions * args.steps / elapsed
    line = {
        'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': 1e3 * elapsed / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'bf16', 'data': 'synthetic', 'impl': 'reference',
        'config': {'workload': workload_name(shape, args), 'linears': 'bf16', 'questions_per_step': arm.questions,
                   'parallelism': 'host cores', 'sample': arm.describe()},
        'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': arm.kind,
                         'sample': arm.describe()},
        'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# op-level timings and library peaks (one GPU)
# --------------------------------------------------------------------------------------

def timed_loop(fn, seconds=0.5, warmup=3):
    """Average ms of `fn`, CUDA events on the current stream, about `seconds` of launches after warm-up."""
    for _ in range(warmup):
        fn()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    iters = int(max(10, min(2000, seconds * 1e3 / max(begin.elapsed_time(end), 1e-3))))
    begin.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / iters


def op_level(device, pk):
    """Config 2 (packed encoder attention, 16 sequences, 35 862 tokens) and config 3 (GeGLU MLP,
    32 768 tokens) with the library peaks measured beside them.  Inputs exceed the 126 MB L2
    (attention: 441 MB of q, k, v, out; MLP: > 700 MB)."""
    from bongard_b200 import ops

    dev = device
    gen = torch.Generator(device=dev).manual_seed(2)

    def randn(*dims, std=1.0):
        return (torch.randn(*dims, device=dev, generator=gen) * std).bfloat16()

    out = {}
    sampler = ClockSampler(device.index or 0).start()
    # library peaks, same loop as everything else
    a, b = randn(8192, 8192), randn(8192, 8192)
    ms = timed_loop(lambda: torch.matmul(a, b))
    out['bf16_matmul_8192'] = {'tflops': 2 * 8192 ** 3 / ms / 1e9, 'what': 'torch.matmul (cuBLAS)'}
    fp8_peak = None
    try:
        a8, b8 = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn).t().contiguous().t()
        one = torch.ones((), device=dev)
        ms = timed_loop(lambda: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
        fp8_peak = 2 * 8192 ** 3 / ms / 1e9
        out['fp8_scaled_mm_8192'] = {'tflops': fp8_peak, 'what': 'torch._scaled_mm e4m3 x e4m3, tensor-wise scales (cuBLASLt)'}
    except Exception as exc:      # a library call outside this package: report, do not fail the bench
        out['fp8_scaled_mm_8192'] = {'tflops': None, 'error': str(exc)[:200]}
    del a, b
    # config 2
    lengths = wl.varlen_lengths(2, 16)
    t, hq, hkv, d = sum(lengths), 8, 4, 256
    positions = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]).to(dev)
    gain = torch.zeros(d, device=dev, dtype=torch.bfloat16)
    for variant, window, theta in (('global', None, 1e6), ('window1024', 1024, 1e4)):
        qkv = randn(t, (hq + 2 * hkv) * d)
        q = qkv[:, :hq * d].view(t, hq, d)
        k = qkv[:, hq * d:(hq + hkv) * d].view(t, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(t, hkv, d)
        ops.qk_norm_rope_(q, k, gain, gain, positions, ops.inv_freq(d, theta, dev))
        plan = ops.make_plan(lengths, window, dev, group=hq // hkv, head_dim=d)
        ms = timed_loop(lambda: ops.varlen_attention(q, k, v, plan, d ** -0.5))
        tflops = 4 * d * hq * plan.pairs / ms / 1e9
        out[f'attention_{variant}'] = {'ms': ms, 'tflops': tflops, 'frac_of_burst_peak': tflops / pk['burst'],
                                       'frac_of_same_run_matmul': tflops / out['bf16_matmul_8192']['tflops'],
                                       'tokens': t, 'algorithmic_tflop': 4 * d * hq * plan.pairs / 1e12}
    # config 3
    t, h, i = 32768, 2560, 10240
    x, wgu, wd = randn(t, h), randn(2 * i, h, std=0.02), randn(h, i, std=0.02)
    flops = 6 * t * h * i
    ms = timed_loop(lambda: ops.linear(ops.linear_geglu(x, wgu), wd))
    out['mlp_bf16'] = {'ms': ms, 'tflops': flops / ms / 1e9, 'frac_of_burst_peak': flops / ms / 1e9 / pk['burst'],
                       'frac_of_same_run_matmul': flops / ms / 1e9 / out['bf16_matmul_8192']['tflops'], 'tokens': t}
    qgu, qd = ops.quantize_weight(wgu), ops.quantize_weight(wd)
    ms = timed_loop(lambda: ops.linear_fp8(ops.linear_fp8(x, qgu, geglu=True), qd))
    out['mlp_fp8_block128'] = {'ms': ms, 'tflops': flops / ms / 1e9, 'includes': 'activation quantisation',
                               'frac_of_fp8_peak': flops / ms / 1e9 / fp8_peak if fp8_peak else None,
                               'speedup_over_bf16': out['mlp_bf16']['ms'] / ms}
    del qgu, qd
    mgu, md = ops.quantize_mxfp8(wgu), ops.quantize_mxfp8(wd)
    ms = timed_loop(lambda: ops.mlp_mxfp8(x, mgu, md))
    out['mlp_mxfp8'] = {'ms': ms, 'tflops': flops / ms / 1e9, 'includes': 'activation quantisation',
                        'frac_of_fp8_peak': flops / ms / 1e9 / fp8_peak if fp8_peak else None,
                        'speedup_over_bf16': out['mlp_bf16']['ms'] / ms}
    # glue at 32768 tokens against the measured copy bandwidth
    y, w = randn(t, h), randn(h, std=0.1)
    for name, fn, nbytes in (('rmsnorm', lambda: ops.rmsnorm(x, w), 2 * t * h * 2),
                             ('add_rmsnorm', lambda: ops.add_rmsnorm_(y, w, x, w), 4 * t * h * 2)):
        ms = timed_loop(fn, seconds=0.2)
        out[name] = {'ms': ms, 'gbs': nbytes / ms / 1e6, 'frac_of_hbm_peak': nbytes / ms / 1e6 / pk['hbm']}
    qkv = randn(t, 4096)
    pos = torch.arange(t, device=dev, dtype=torch.int32) % 4096
    gain = randn(256, std=0.1)
    freqs = ops.inv_freq(256, 1e4, dev)
    ms = timed_loop(lambda: ops.qk_norm_rope_(qkv[:, :2048].view(t, 8, 256), qkv[:, 2048:3072].view(t, 4, 256), gain, gain,
                                              pos, freqs), seconds=0.2)
    out['qk_norm_rope_sincos'] = {'ms': ms, 'gbs': 2 * t * 3072 * 2 / ms / 1e6, 'frac_of_hbm_peak': 2 * t * 3072 * 2 / ms / 1e6 / pk['hbm']}
    table = ops.rope_table(256, 1e4, 4096, dev)      # the form the packed engine runs: angles from a per-position table
    ms = timed_loop(lambda: ops.qk_norm_rope_(qkv[:, :2048].view(t, 8, 256), qkv[:, 2048:3072].view(t, 4, 256), gain, gain,
                                              pos, None, table=table), seconds=0.2)
    out['qk_norm_rope'] = {'ms': ms, 'gbs': 2 * t * 3072 * 2 / ms / 1e6, 'frac_of_hbm_peak': 2 * t * 3072 * 2 / ms / 1e6 / pk['hbm']}
    out['clocks'] = sampler.stop()
    out['peaks'] = {'bf16_burst_tflops': pk['burst'], 'hbm_gbs': pk['hbm'], 'source': pk['source']}
    return out


# --------------------------------------------------------------------------------------
# the B200 arm
# --------------------------------------------------------------------------------------

def run_b200(args):
    import torch.distributed as dist

    from bongard_b200 import ops
    from bongard_b200.engine import JudgmentEngine

    world, rank, local = dist_setup()
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    shape = wl.SHAPES[args.shape]
    weights = wl.make_weights_device(shape, args.seed, device)

    def build(linears):
        e = JudgmentEngine(weights, shape, device, linears=linears, encoder_pack_tokens=args.encoder_pack_tokens,
                           decoder_pack_tokens=args.decoder_pack_tokens, residual='bf16' if linears == 'mxfp8' else args.residual[:4], wide_outputs=args.residual.endswith('wide'))
        e.programmatic_launch = args.programmatic_launches
        return e

    engine = build(args.linears)
    requests = make_requests(shape, args.seed + rank, args.requests, args.workload)
    questions = sum(len(r.questions) for r in requests)
    batch = engine.prepare(requests)
    staged, offsets = engine.stage(batch)
    max_candidates = 10 * 64 * max(args.requests, 4)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gather(probs):
        """Answers to rank 0: one fixed-size all_gather of float64 probabilities."""
        if world == 1:
            return probs
        padded = torch.zeros(max_candidates, device=device, dtype=torch.float64)
        padded[:probs.numel()] = probs
        out = torch.empty(world * max_candidates, device=device, dtype=torch.float64)
        dist.all_gather_into_tensor(out, padded)
        return out

    def device_step():
        return gather(engine.probabilities(engine.execute(staged), offsets))

    def host_step():
        b = engine.prepare(requests)
        st, off = engine.stage(b)
        return gather(engine.probabilities(engine.execute(st), off)).cpu()

    for _ in range(args.warmup):
        device_step()
    barrier()

    # ---- timed: kernels over HBM-resident inputs
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ops.GEMM_TIMER, ops.ATTN_TIMER = ops.KernelTimer(), ops.KernelTimer()
    launches0 = engine.launches
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    begin.record()
    for _ in range(args.steps):
        device_step()
    end.record()
    barrier()
    device_ms = begin.elapsed_time(end)
    launches = (engine.launches - launches0) // args.steps
    gemm_ms, attn_ms = ops.GEMM_TIMER.total_ms(), ops.ATTN_TIMER.total_ms()
    gemm_flops, attn_flops, gemm_launches = ops.GEMM_TIMER.flops, ops.ATTN_TIMER.flops, ops.GEMM_TIMER.launches
    ops.GEMM_TIMER = ops.ATTN_TIMER = None

    # ---- timed: end to end from host request objects
    host_step()
    barrier()
    begin.record()
    for _ in range(args.steps):
        host = host_step()
    end.record()
    barrier()
    e2e_ms = begin.elapsed_time(end)
    clocks = sampler.stop() if sampler else None
    ops.read_status()

    times = torch.tensor([device_ms, e2e_ms], device=device, dtype=torch.float64)
    counts = torch.tensor([float(questions)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
    device_ms, e2e_ms = times.tolist()
    total_questions = counts.item()
    full_answers = host[:sum(batch.sizes)].clone() if rank == 0 else None     # rank 0's batch is the seed-`args.seed` batch
    del staged, offsets, host

    extras = {}
    if not args.no_extras and shape.name != 'tiny':
        if world > 1 and args.workload == 'judged':
            extras['strong'] = strong_scaling(args, engine, shape, device, world, rank, full_answers, barrier)
        if args.workload == 'judged':
            extras['long_context'] = long_context(args, build, engine, shape, device, world, rank, barrier)
    del weights

    if rank == 0:
        pk = peaks()
        achieved = gemm_flops / gemm_ms / 1e9
        line = {
            'metric': METRIC, 'value': total_questions * args.steps / (device_ms / 1e3), 'unit': UNIT, 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': device_ms / args.steps, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {
                'workload': workload_name(shape, args), 'linears': args.linears, 'residual_stream': args.residual,
                'questions_per_step': int(total_questions), 'parallelism': f'dp{world}',
                'packs': f'states in encoder packs of up to {args.encoder_pack_tokens} tokens, whole 8-question decoder groups '
                         f'in packs of up to {args.decoder_pack_tokens} tokens',
                'l2': 'inputs larger than L2: 14 GB of weights and >1 GB of activations stream per layer',
                'tflop_per_step_per_gpu': (batch.gemm_flops + batch.attn_flops) / 1e12,
            },
            'e2e': {'value': total_questions * args.steps / (e2e_ms / 1e3), 'unit': UNIT,
                    'h2d_bytes_per_step': batch.h2d_bytes, 'd2h_bytes_per_step': int(max_candidates * world * 8 if world > 1 else sum(batch.sizes) * 8)},
            'gpu_launches': int(launches),
            'roofline': {'bound': 'tensor',
                         'kernel': {'bf16': 'gemm_bf16_pair_kernel', 'fp8': 'gemm_fp8_kernel', 'mxfp8': 'gemm_mxfp8_kernel'}[args.linears],
                         'achieved': achieved, 'peak': pk['sustained'],
                         'unit': 'TFLOP/s', 'frac': achieved / pk['sustained'], 'peak_source': pk['source'] + ' sustained',
                         'launches': gemm_launches, 'share_of_step': gemm_ms / device_ms,
                         'traffic': GEMM_TRAFFIC_PER_FLOP * gemm_flops / gemm_launches,
                         'traffic_source': 'scaled by FLOPs from an ncu capture of the 8192-token MLP GEMMs, '
                                           'not measured on these launches'},
            'attention': {'achieved': attn_flops / attn_ms / 1e9 if attn_ms else None, 'unit': 'TFLOP/s',
                          'frac': attn_flops / attn_ms / 1e9 / pk['sustained'] if attn_ms else None,
                          'peak_source': pk['source'] + ' sustained', 'share_of_step': attn_ms / device_ms},
            'model_tflops': (batch.gemm_flops + batch.attn_flops) * args.steps / device_ms / 1e9,
            'clocks': clocks,
        }
        line.update(extras)
        if world == 1 and not args.no_extras and shape.name != 'tiny':
            del engine
            torch.cuda.empty_cache()
            line['ops'] = op_level(device, pk)
            engine = None
        if world == 1 and not args.no_cpu_baseline:
            cpu_weights = {name: t.cpu() for name, t in wl.make_weights_device(shape, args.seed, device).items()}
            arm = CpuArm(shape, cpu_weights, requests, args.cpu_seconds)
            del cpu_weights
            seconds = arm.step()
            line['cpu_baseline'] = {'value': arm.questions / seconds, 'unit': UNIT, 'cores': torch.get_num_threads(),
                                    'kind': arm.kind, 'sample': arm.describe(), 'seconds': seconds}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def strong_scaling(args, engine, shape, device, world, rank, full_answers, barrier):
    """ONE batch (seed `args.seed`, `args.requests` requests) split over the ranks with the
    longest-processing-time-first rule; every rank computes the assignment locally.  Returns
    (rank 0) throughput, per-rank times and the comparison of the gathered answers with rank 0's
    own answers for the whole batch."""
    import torch.distributed as dist

    requests = make_requests(shape, args.seed, args.requests, args.workload)
    costs = [wl.fast_request_cost(shape, r) for r in requests]
    shards = wl.partition_requests(costs, world)
    mine = [requests[i] for i in shards[rank]]
    batch = engine.prepare(mine)
    staged, offsets = engine.stage(batch)
    per_rank = 10 * 64 * ((args.requests + world - 1) // world + 8)

    def step():
        probs = engine.probabilities(engine.execute(staged), offsets)
        padded = torch.zeros(per_rank, device=device, dtype=torch.float64)
        padded[:probs.numel()] = probs
        out = torch.empty(world * per_rank, device=device, dtype=torch.float64)
        dist.all_gather_into_tensor(out, padded)
        return out, probs

    step()
    sampler = ClockSampler(device.index or 0).start() if rank == 0 else None
    begin, end, mid = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    steps = max(1, args.extra_steps)
    own_ms = 0.0
    barrier()
    begin.record()
    for _ in range(steps):
        mid.record()
        probs = engine.probabilities(engine.execute(staged), offsets)
        done = torch.cuda.Event(enable_timing=True)
        done.record()
        padded = torch.zeros(per_rank, device=device, dtype=torch.float64)
        padded[:probs.numel()] = probs
        gathered = torch.empty(world * per_rank, device=device, dtype=torch.float64)
        dist.all_gather_into_tensor(gathered, padded)
        torch.cuda.synchronize()
        own_ms += mid.elapsed_time(done)
    end.record()
    barrier()
    total = torch.tensor([begin.elapsed_time(end)], device=device, dtype=torch.float64)
    dist.all_reduce(total, op=dist.ReduceOp.MAX)
    each = torch.zeros(world, device=device, dtype=torch.float64)
    each[rank] = own_ms / steps
    dist.all_reduce(each, op=dist.ReduceOp.SUM)
    clocks = sampler.stop() if sampler else None
    if rank != 0:
        return None
    # put the gathered answers back into request order and compare with the whole-batch run
    restored = wl.reassemble_answers(gathered.cpu(), shards, requests, per_rank)
    diff = float((restored - full_answers).abs().max()) if restored.numel() == full_answers.numel() else None
    each = each.tolist()
    questions = sum(len(r.questions) for r in requests)
    return {'value': questions * steps / (total.item() / 1e3), 'unit': UNIT, 'steps': steps, 'ms_per_step': total.item() / steps,
            'requests': len(requests), 'questions': questions, 'partition': 'longest processing time first over a closed-form FLOP cost',
            'rank_ms': each, 'imbalance': max(each) / (sum(each) / len(each)),
            'answers_bit_equal_to_one_gpu_run': bool(diff == 0.0), 'answers_max_abs_diff': diff, 'clocks': clocks}


def long_context(args, build, engine, shape, device, world, rank, barrier):
    """32 768-token states with 64 questions each, 4 requests per GPU (32 over 8 GPUs), in bf16 and
    with both FP8 recipes for the projections and the MLP."""
    import torch.distributed as dist

    requests = wl.long_context_requests(5 + rank, vocab=shape.vocab, requests=4, eoi=shape.eoi_token)
    questions = sum(len(r.questions) for r in requests)
    out = {'requests_per_gpu': 4, 'state_tokens': 32768, 'questions_per_request': 64, 'unit': UNIT}
    steps = max(1, args.extra_steps)
    for linears in ('bf16', 'fp8', 'mxfp8'):
        e = engine if linears == engine.linears else build(linears)
        batch = e.prepare(requests)
        staged, offsets = e.stage(batch)
        e.probabilities(e.execute(staged), offsets)
        sampler = ClockSampler(device.index or 0).start() if rank == 0 else None
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        begin.record()
        for _ in range(steps):
            e.probabilities(e.execute(staged), offsets)
        end.record()
        barrier()
        ms = torch.tensor([begin.elapsed_time(end)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        clocks = sampler.stop() if sampler else None
        out[linears] = {'value': questions * world * steps / (ms.item() / 1e3), 'ms_per_step': ms.item() / steps, 'steps': steps,
                        'model_tflops': (batch.gemm_flops + batch.attn_flops) * steps / ms.item() / 1e9, 'clocks': clocks}
        del staged, offsets, batch
        if e is not engine:
            del e
            torch.cuda.empty_cache()
    return out if rank == 0 else None


def main():
    args = parse()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_b200(args)


if __name__ == '__main__':
    main()
