"""One rank of the two-GPU tensor-parallel check (started by test_gpu_i_tp.py through
torch.distributed.run): the same utterance decoded single-GPU and tensor-parallel must give the
same codes on every rank, and the library must return to single-GPU launches after tp_close."""
import ctypes as C
import os
import sys

import numpy as np

rank = int(os.environ["RANK"])
world = int(os.environ["WORLD_SIZE"])
os.environ["VB200_DEVICE"] = os.environ.get("LOCAL_RANK", "0")

import torch.distributed as dist  # noqa: E402

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from conftest import load_package  # noqa: E402


def main():
    dist.init_process_group("gloo")
    pkg = load_package()
    model = pkg.SynthModel()
    eng = pkg.Engine(256)
    eng.upload(model, decoder=True, acoustic=True, audio_table=True)
    L = eng.L
    frames = 6
    prompt = pkg.synth_f32((40, 3072), 3, "tp.prompt", 0.0, 0.5)
    noise = pkg.synth_f32((frames, 36), 4, "tp.noise")
    first = model.token_rows([24])[0]

    def run():
        eng.prefill(prompt, 0)
        codes, _, _ = eng.utterance(first, 40, noise)
        return codes

    want = run()
    handle = (C.c_ubyte * 64)()
    assert L.vb200_tp_arena(rank, world, handle) == 0
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle))
    assert L.vb200_tp_connect(b"".join(handles)) == 0
    dist.barrier()
    got = run()
    got2 = run()                      # second run replays the captured graph
    dist.barrier()
    L.vb200_tp_close()
    after = run()
    ok = np.array_equal(want, got) and np.array_equal(want, got2) and np.array_equal(want, after)
    ok = ok and L.vb200_last_status() == 0
    print(f"rank {rank}: {'OK' if ok else 'MISMATCH'}", flush=True)
    eng.close()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
