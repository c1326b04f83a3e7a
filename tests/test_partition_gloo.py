"""Data-parallel request partition and answer gather with world-size-2 gloo ranks on CPU."""

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bongard_b200 import workload as wl


def test_partition_is_balanced_and_complete():
    requests = wl.judged_requests(4, requests=64, with_ids=False)
    costs = [wl.fast_request_cost(wl.B4, r) for r in requests]
    for world in (1, 2, 4, 8):
        shards = wl.partition_requests(costs, world)
        assert sorted(i for s in shards for i in s) == list(range(len(requests)))
        loads = [sum(costs[i] for i in s) for s in shards]
        assert max(loads) <= 1.08 * (sum(costs) / world)
        assert shards == wl.partition_requests(costs, world)        # deterministic on every rank


def test_cost_model_tracks_exact_flops():
    requests = wl.judged_requests(7, requests=6, state=(512, 2048), with_ids=False)
    for r in requests:
        exact, fast = wl.request_flops(wl.B4, r), wl.fast_request_cost(wl.B4, r)
        assert abs(fast - exact) / exact < 0.05


def _rank(rank, world, port, out):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    requests = wl.tiny_requests(3, requests=7, questions=2)
    shards = wl.partition_requests([wl.fast_request_cost(wl.TINY, r) for r in requests], world)
    mine = shards[rank]
    # stand-in for the judged probabilities: a value derived from (request, question, candidate)
    flat = torch.tensor([i * 100 + j * 10 + c for i in mine for j, q in enumerate(requests[i].questions.values())
                         for c in range(len(q.candidate_positions))], dtype=torch.float64)
    width = 7 * 2 * 5
    padded = torch.zeros(width, dtype=torch.float64)
    padded[:flat.numel()] = flat
    gathered = [torch.zeros(width, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, padded)
    if rank == 0:
        # the flat reassembly the benchmark uses for its strong-scaling check
        whole = wl.reassemble_answers(torch.cat(gathered), shards, requests, width)
        expect = [i * 100 + j * 10 + c for i in range(len(requests)) for j, q in enumerate(requests[i].questions.values())
                  for c in range(len(q.candidate_positions))]
        assert whole.tolist() == [float(v) for v in expect]
        answers = {}
        for r, buf in enumerate(gathered):
            cursor = 0
            for i in shards[r]:
                for j, q in enumerate(requests[i].questions.values()):
                    n = len(q.candidate_positions)
                    answers[(i, j)] = buf[cursor:cursor + n].tolist()
                    cursor += n
        torch.save(answers, out)
    dist.barrier()
    dist.destroy_process_group()


def test_gather_reassembles_every_answer(tmp_path):
    out = tmp_path / 'answers.pt'
    mp.spawn(_rank, args=(2, 29541, str(out)), nprocs=2, join=True)
    answers = torch.load(out)
    requests = wl.tiny_requests(3, requests=7, questions=2)
    assert len(answers) == 14
    for (i, j), values in answers.items():
        q = list(requests[i].questions.values())[j]
        assert values == [float(i * 100 + j * 10 + c) for c in range(len(q.candidate_positions))]
