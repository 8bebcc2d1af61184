"""Tensor-parallel token loop on CPU ranks: world_size 2 and 4 over torch.distributed (gloo), every rank running its
shard of the tiny model on the CPU oracle backend.  The gathered logits and the greedy tokens must equal the
single-rank model bit for bit (sharding copies finished values only, so it cannot change a bit)."""
import ctypes as C
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
SEED = 20261125


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_rank(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    from det_b200 import capi
    os.environ["OMP_NUM_THREADS"] = "2"
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    h = capi.host()
    o = C.CDLL(str(ROOT / "oracle" / "_build" / "liboracle.so"))
    o.orc_ref_backend_new.restype = C.c_void_p
    backend = o.orc_ref_backend_new()

    @C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_size_t)
    def gather(local, gathered, nbytes):
        src = torch.from_numpy(np.ctypeslib.as_array(C.cast(local, C.POINTER(C.c_uint8)), shape=(nbytes,)).copy())
        parts = [torch.empty(nbytes, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(parts, src)
        dst = np.ctypeslib.as_array(C.cast(gathered, C.POINTER(C.c_uint8)), shape=(world * nbytes,))
        dst[:] = torch.cat(parts).numpy()

    comm = h.dh_callback_comm_new(rank, world, C.cast(gather, C.c_void_p))
    ids = np.zeros(6, np.int32)
    h.dh_synth_prompt(1, 6, 32768, ids.ctypes.data)

    def run(model):
        assert h.dh_model_prefill(model, ids.ctypes.data, 4) == 0, h.dh_last_error()   # a 4-token batch ...
        assert h.dh_model_forward(model, ids[4:].ctypes.data, 2) == 0, h.dh_last_error()   # ... then a 2-token one
        toks = np.zeros(3, np.int32)
        n = C.c_size_t(0)
        assert h.dh_model_generate(model, ids.ctypes.data, 0, 3, 1, 1.0, 0, 1.0, 0, toks.ctypes.data, C.byref(n)) == 0
        logits = np.zeros(32768, np.float32)
        h.dh_model_logits(model, logits.ctypes.data, logits.size)
        return toks.copy(), logits.view(np.uint32).copy()

    shard = h.dh_model_new_synth_tp(backend, b"tiny", 4, SEED, 32, 4, comm)
    assert shard, h.dh_last_error()
    got = run(shard)
    if rank == 0:
        full = h.dh_model_new_synth(backend, b"tiny", 4, SEED, 32, 4)
        want = run(full)
        np.savez(Path(out_dir) / "result.npz", tok_ok=np.array_equal(got[0], want[0]),
                 logit_diff=int((got[1] != want[1]).sum()), toks=got[0])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_model_equals_single_rank(world, libs, oracle, tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_run_rank, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = np.load(tmp_path / "result.npz")
    assert int(r["logit_diff"]) == 0, f"{int(r['logit_diff'])} logits differ between world_size {world} and 1"
    assert bool(r["tok_ok"])


def _run_rank_serving(rank, world, port, out_dir):
    """Three sequences of different prompt lengths advance together on a sharded model (each rank holds its heads'
    caches and states of every sequence); rank 0 also produces every stream alone on the unsharded model."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    from det_b200 import capi
    os.environ["OMP_NUM_THREADS"] = "2"
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    h = capi.host()
    o = C.CDLL(str(ROOT / "oracle" / "_build" / "liboracle.so"))
    o.orc_ref_backend_new.restype = C.c_void_p
    backend = o.orc_ref_backend_new()

    @C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_size_t)
    def gather(local, gathered, nbytes):
        src = torch.from_numpy(np.ctypeslib.as_array(C.cast(local, C.POINTER(C.c_uint8)), shape=(nbytes,)).copy())
        parts = [torch.empty(nbytes, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(parts, src)
        dst = np.ctypeslib.as_array(C.cast(gathered, C.POINTER(C.c_uint8)), shape=(world * nbytes,))
        dst[:] = torch.cat(parts).numpy()

    comm = h.dh_callback_comm_new(rank, world, C.cast(gather, C.c_void_p))
    prompts, n_new = [5, 11, 3], 5
    sampling = (0, 1.0 / 0.7, 40, 0.95)

    def prompt(i, n):
        ids = np.zeros(n, np.int32)
        h.dh_synth_prompt(100 + i, n, 32768, ids.ctypes.data)
        return ids

    shard = h.dh_model_new_synth_tp(backend, b"tiny", 4, SEED, 48, 8, comm)
    assert shard, h.dh_last_error()
    batch = h.dh_batch_new(shard, len(prompts), 48)
    assert batch, h.dh_last_error()
    for i, n in enumerate(prompts):
        ids = prompt(i, n)          # held in a name: the pointer of a temporary dies with it
        assert h.dh_batch_prefill(batch, i, ids.ctypes.data, n, *sampling, 7000 + i) == 0, h.dh_last_error()
    assert h.dh_batch_step(batch, n_new - 1) == 0, h.dh_last_error()
    together = []
    for i in range(len(prompts)):
        out = np.zeros(n_new, np.int32)
        assert h.dh_batch_tokens(batch, i, out.ctypes.data, n_new) == n_new
        together.append(out)
    if rank == 0:
        full = h.dh_model_new_synth(backend, b"tiny", 4, SEED, 48, 8)
        ok = True
        for i, n in enumerate(prompts):
            out = np.zeros(n_new, np.int32)
            cnt = C.c_size_t(0)
            assert h.dh_model_reset(full) == 0
            ids = prompt(i, n)
            assert h.dh_model_generate(full, ids.ctypes.data, n, n_new, *sampling, 7000 + i, out.ctypes.data,
                                       C.byref(cnt)) == 0, h.dh_last_error()
            ok = ok and cnt.value == n_new and np.array_equal(out, together[i])
        np.savez(Path(out_dir) / "serving.npz", ok=ok, streams=np.stack(together))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_serving_streams_equal_solo_streams(libs, oracle, tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_run_rank_serving, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r = np.load(tmp_path / "serving.npz")
    assert bool(r["ok"]), r["streams"]
