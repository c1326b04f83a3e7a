"""Judged questions per second at the 4B-4B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one pass of the whole hot path (encoder over every state, state K/V projection,
decoder over every question, judgment head, candidate softmax) over one batch of seeded
synthetic requests: 256 requests, states of 512-8192 tokens, 1-24 questions each.  Every rank
holds a full bf16 replica and its own batch (rank r uses seed 4 + r), so scaling is weak; the
only collective is the gather of answers.

`value` times the kernels with the batch already staged in HBM; `e2e` times the public
call JudgmentEngine.judge() from host request objects (host layout, pinned copies, kernels,
one device-to-host copy of the probabilities).  The dominant kernel (the BF16 tensor-core
GEMM) is timed live with CUDA events for the roofline entry.  `--impl reference` times the
CPU restatement of the reference's own path on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from bongard_b200 import workload as wl  # noqa: E402

METRIC = 'judged_questions_per_second'
UNIT = 'questions/s'
# DRAM bytes per algorithmic FLOP of the GEMM, from the ncu capture of the 8192-token MLP GEMMs (scaled to a launch by its FLOPs)
GEMM_TRAFFIC_PER_FLOP = 7.0e-4    # (337.5 + 565.1) MB over (0.859 + 0.429) TFLOP, profiles/gemm_bf16_mlp_8192tokens.md


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
                    help='launch kernels with programmatic stream serialization (no effect on throughput: 297.5 vs 297.1)')
    ap.add_argument('--linears', default='bf16', choices=['bf16', 'fp8', 'mxfp8'], help='projection / MLP GEMM precision')
    ap.add_argument('--cpu-seconds', type=float, default=15.0, help='CPU baseline budget per sample')
    ap.add_argument('--encoder-pack-tokens', type=int, default=65536)
    ap.add_argument('--decoder-pack-tokens', type=int, default=16384)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    args = ap.parse_args()
    if args.seed is None:
        args.seed = 5 if args.workload == 'long' else 4
    if args.workload == 'long' and args.requests == 256:
        args.requests = 4          # four 32768-token states with 64 questions each per GPU
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


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""

    FIELDS = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, f'/tmp/bg_clocks_{os.getpid()}.csv'

    def start(self):
        try:
            self.out = open(self.path, 'w')
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}',
                                          '--format=csv,noheader,nounits', '-lms', '200'], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        self.proc.wait()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in open(self.path):
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith('active'):
                    reasons.add(name)
        os.unlink(self.path)
        sm.sort()
        return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'samples': len(sm), 'reasons': sorted(reasons)}


# --------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's device="cpu" path
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


def cpu_sample(shape, requests, budget_seconds):
    """The cheapest requests of the batch, with as many of their questions as fit a FLOP budget
    derived from a one-second matmul calibration."""
    rate = cpu_matmul_tflops(torch.bfloat16) * 1e12 * 0.5       # the whole path runs at about half of matmul peak
    budget = rate * budget_seconds
    order = sorted(range(len(requests)), key=lambda i: wl.fast_request_cost(shape, requests[i]))
    chosen, spent = [], 0.0
    for i in order:
        r = requests[i]
        cost = wl.fast_request_cost(shape, r)
        if chosen and spent + cost > budget:
            break
        if not chosen and cost > budget:
            # trim the questions of the cheapest request rather than run over budget
            qs = dict(list(r.questions.items())[:max(1, int(len(r.questions) * budget / cost))])
            r = wl.Request(r.state, qs, r.input_tokens)
        chosen.append(r)
        spent += cost
    return chosen


def cpu_run(shape, weights, sample):
    from oracle import reference_math as om

    with torch.inference_mode():
        t0 = time.perf_counter()
        result = om.forward_packed(weights, shape, sample, 8, dtype=torch.bfloat16)
        for answers in result:
            for v in answers.values():
                om.probabilities(v['logits'].float())
        return time.perf_counter() - t0


def describe(sample):
    return (f'{len(sample)} cheapest request(s) of the step batch: {sum(len(r.state) for r in sample)} state tokens, '
            f'{sum(len(r.questions) for r in sample)} questions, bf16, torch CPU with {torch.get_num_threads()} threads')


# --------------------------------------------------------------------------------------
# arms
# --------------------------------------------------------------------------------------

def dist_setup(args):
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    return world, rank, local


def run_reference(args):
    """The reference's CPU path (oracle port) on the host cores; rank 0 only."""
    world, rank, _ = dist_setup(args)
    if rank != 0:
        return
    shape = wl.SHAPES[args.shape]
    torch.set_num_threads(os.cpu_count() or 1)
    gen = torch.Generator().manual_seed(args.seed)
    weights = {name: (torch.randn(dims, generator=gen, dtype=torch.bfloat16) * (0.02 if len(dims) >= 2 else 0.0))
               for name, dims in wl.weight_names(shape)}
    requests = make_requests(shape, args.seed, args.requests, args.workload)
    sample = cpu_sample(shape, requests, args.cpu_seconds)
    questions = sum(len(r.questions) for r in sample)
    for _ in range(args.warmup):
        cpu_run(shape, weights, sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_run(shape, weights, sample)
    elapsed = time.perf_counter() - t0
    value = questions * args.steps / elapsed
    line = {
        'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': 1e3 * elapsed / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'bf16', 'data': 'synthetic', 'impl': 'reference',
        'config': {'workload': f'{shape.name} judged requests, seed {args.seed}: bounded sample per step', 'sample': describe(sample)},
        'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port', 'sample': describe(sample)},
        'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


def run_b200(args):
    import torch.distributed as dist

    from bongard_b200 import ops
    from bongard_b200.engine import JudgmentEngine

    world, rank, local = dist_setup(args)
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    shape = wl.SHAPES[args.shape]
    weights = wl.make_weights_device(shape, args.seed, device)
    engine = JudgmentEngine(weights, shape, device, linears=args.linears, encoder_pack_tokens=args.encoder_pack_tokens,
                            decoder_pack_tokens=args.decoder_pack_tokens)
    engine.programmatic_launch = args.programmatic_launches
    del weights
    requests = make_requests(shape, args.seed + rank, args.requests, args.workload)
    questions = sum(len(r.questions) for r in requests)
    batch = engine.prepare(requests)
    staged, offsets = engine.stage(batch)
    max_candidates = 10 * 64 * args.requests

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
    if rank == 0:
        pk = peaks()
        achieved = gemm_flops / gemm_ms / 1e9
        line = {
            'metric': METRIC, 'value': total_questions * args.steps / (device_ms / 1e3), 'unit': UNIT, 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': device_ms / args.steps, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {
                'workload': (f'{shape.name} judged requests: {args.requests} requests per GPU per step, states 512-8192 tokens, '
                             f'1-24 questions each, 8 questions per decoder group (seed {args.seed} + rank)'
                             if args.workload == 'judged' else
                             f'{shape.name} long-context shared evidence: {args.requests} requests per GPU per step, 32768-token '
                             f'states, 64 questions each in groups of 8 (seed {args.seed} + rank)'),
                'linears': args.linears,
                'questions_per_step': int(total_questions), 'parallelism': f'dp{world}',
                'l2': 'inputs larger than L2: 14 GB of weights and >1 GB of activations stream per layer',
                'tflop_per_step_per_gpu': (batch.gemm_flops + batch.attn_flops) / 1e12,
            },
            'e2e': {'value': total_questions * args.steps / (e2e_ms / 1e3), 'unit': UNIT,
                    'h2d_bytes_per_step': batch.h2d_bytes, 'd2h_bytes_per_step': int(host.numel() * 8)},
            'gpu_launches': int(launches),
            'roofline': {'bound': 'tensor', 'kernel': {'bf16': 'gemm_bf16_pair_kernel', 'fp8': 'gemm_fp8_kernel', 'mxfp8': 'gemm_mxfp8_kernel'}[args.linears], 'achieved': achieved, 'peak': pk['sustained'],
                         'unit': 'TFLOP/s', 'frac': achieved / pk['sustained'], 'peak_source': pk['source'] + ' sustained',
                         'launches': gemm_launches, 'share_of_step': gemm_ms / device_ms,
                         'traffic': None if GEMM_TRAFFIC_PER_FLOP is None else GEMM_TRAFFIC_PER_FLOP * gemm_flops / gemm_launches},
            'attention': {'achieved': attn_flops / attn_ms / 1e9 if attn_ms else None, 'unit': 'TFLOP/s',
                          'frac': attn_flops / attn_ms / 1e9 / pk['sustained'] if attn_ms else None,
                          'share_of_step': attn_ms / device_ms},
            'model_tflops': (batch.gemm_flops + batch.attn_flops) * args.steps / device_ms / 1e9,
            'clocks': clocks,
        }
        if not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            cpu_weights = {name: t.cpu() for name, t in wl.make_weights_device(shape, args.seed, device).items()}
            sample = cpu_sample(shape, requests, args.cpu_seconds)
            seconds = cpu_run(shape, cpu_weights, sample)
            line['cpu_baseline'] = {'value': sum(len(r.questions) for r in sample) / seconds, 'unit': UNIT,
                                    'cores': torch.get_num_threads(), 'kind': 'port', 'sample': describe(sample),
                                    'seconds': seconds}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_b200(args)


if __name__ == '__main__':
    main()
