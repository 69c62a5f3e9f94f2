"""The N > 1 host logic of bench.py on CPU: two gloo ranks, independent utterances per rank,
whole-job throughput = all ranks' frames / the slowest rank's time."""
import importlib.util
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    bench = _bench()
    seeds = bench.utterance_seeds(rank)
    local_ms = 100.0 * (rank + 1)                 # rank 1 is the slow one
    value, max_ms = bench.aggregate(local_ms, 50, dist, device="cpu")
    shared_value, _ = bench.aggregate(local_ms, 50, dist, device="cpu", shared=True)
    assert abs(shared_value * world - value) < 1e-9      # the same frames on every rank count once
    gathered = [None] * world
    dist.all_gather_object(gathered, seeds)
    if rank == 0:
        out.put((value, max_ms, gathered))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_aggregate_and_shard():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    value, max_ms, seeds = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert max_ms == 200.0                        # the slowest rank's time
    assert abs(value - 2 * 50 / 0.2) < 1e-9       # all frames over that time
    assert seeds[0] != seeds[1]                   # every rank works on its own utterance
    assert seeds[0] == {"prompt": 100, "noise": 1000}


def test_single_rank_aggregate():
    bench = _bench()
    value, ms = bench.aggregate(4.0, 2, None, device="cpu")
    assert ms == 4.0 and abs(value - 500.0) < 1e-9
    # tensor parallelism: all ranks worked on the same frames, which therefore count once
    value, ms = bench.aggregate(4.0, 2, None, device="cpu", shared=True)
    assert abs(value - 500.0) < 1e-9


def test_frame_bytes_match_survey_figures():
    bench = _bench()
    # decoder step at 65 keys: 26 * W_layer + norms + KV read + KV write (6.067 GB)
    dec64 = bench.LLM_WEIGHT_BYTES + bench.LLM_NORM_BYTES + 26 * 65 * 8192 + bench.KV_WRITE_BYTES
    assert bench.LLM_WEIGHT_BYTES == 6_052_380_672
    assert abs(dec64 - 6.067e9) < 2e6
    assert bench.frame_bytes(64) == dec64 + bench.ACOUSTIC_BYTES + bench.REEMBED_BYTES
