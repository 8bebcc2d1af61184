"""Tensor-parallel token loop on real GPUs (one process per GPU): the shard of every rank runs on the CUDA backend, decode
exchanges go through the peer-memory kernels (fused with their consumer, det_xchg_add_rmsnorm_quant / det_xchg_quant, or
stand-alone, det_xchg_all_gather), the 16-token batch through NCCL.  Logits and greedy
tokens must equal the single-GPU model bit for bit, eagerly and through the captured decode graph.  Skipped on a box
with fewer GPUs than ranks."""
import ctypes as C
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
SEED = 20261125
VOCAB = 32768


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_rank(rank, world, port, out_dir, exchange):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    from det_b200 import capi
    rt = C.CDLL("libcudart.so.12")
    assert rt.cudaSetDevice(rank) == 0
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    h, d = capi.host(), capi.cuda()
    backend = h.dh_cuda_backend_new(1, 1)
    assert backend, h.dh_last_error()
    nid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = np.zeros(128, np.uint8)
        h.dh_nccl_unique_id(buf.ctypes.data)
        nid = torch.from_numpy(buf)
    dist.broadcast(nid, 0)
    nid_np = nid.numpy().copy()
    if exchange == "nccl":
        comm = h.dh_nccl_comm_new(nid_np.ctypes.data, rank, world)
        assert comm, h.dh_last_error()
    else:
        comm = h.dh_peer_comm_new(nid_np.ctypes.data, rank, world, 16 * max(8 * 3072, VOCAB) + 4096)
        assert comm, h.dh_last_error()
        mine = np.zeros(64, np.uint8)
        h.dh_peer_comm_handle(comm, mine.ctypes.data)
        every = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(every, torch.from_numpy(mine))
        handles = np.concatenate([e.numpy() for e in every]).copy()
        h.dh_peer_comm_open(comm, handles.ctypes.data)
        if exchange == "peer_unfused":
            h.dh_peer_comm_set_fuse(comm, 0)
        dist.barrier()
    ids = np.zeros(22, np.int32)
    h.dh_synth_prompt(1, ids.size, VOCAB, ids.ctypes.data)

    def run(model):
        assert h.dh_model_prefill(model, ids.ctypes.data, 4) == 0, h.dh_last_error()          # 4 rows: peer kernel
        assert h.dh_model_forward(model, ids[4:].ctypes.data, 16) == 0, h.dh_last_error()     # 16 rows: bulk path
        assert h.dh_model_forward(model, ids[20:].ctypes.data, 2) == 0, h.dh_last_error()
        logits = np.zeros(VOCAB, np.float32)
        h.dh_model_logits(model, logits.ctypes.data, logits.size)
        tok = C.c_int32(0)
        rng = C.c_uint64(0)
        assert h.dh_model_pick(model, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(tok)) == 0
        dec = h.dh_graph_decoder_new(model)
        assert dec, h.dh_last_error()
        out = np.zeros(12, np.int32)
        assert h.dh_graph_decoder_enqueue(dec, tok.value, 12, 1) == 0, h.dh_last_error()   # step 1 eager, 11 replays
        n = h.dh_graph_decoder_finish(dec, out.ctypes.data, out.size)
        h.dh_graph_decoder_free(dec)
        return np.concatenate([[tok.value], out[:n]]), logits.view(np.uint32).copy()

    shard = h.dh_model_new_synth_tp(backend, b"tiny", 4, SEED, 64, 16, comm)
    assert shard, h.dh_last_error()
    got = run(shard)
    assert d.det_last_error() == 0
    if rank == 0:
        full = h.dh_model_new_synth(backend, b"tiny", 4, SEED, 64, 16)
        want = run(full)
        np.savez(Path(out_dir) / "result.npz", toks=got[0], want=want[0], logit_diff=int((got[1] != want[1]).sum()))
    d.det_sync()
    dist.barrier()
    dist.destroy_process_group()


def _gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.gpu
@pytest.mark.parametrize("world,exchange", [(2, "peer"), (2, "peer_unfused"), (2, "nccl"), (4, "peer")])
def test_sharded_model_equals_single_gpu(world, exchange, libs, tmp_path):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_run_rank, args=(world, _free_port(), str(tmp_path), exchange), nprocs=world, join=True)
    r = np.load(tmp_path / "result.npz")
    assert int(r["logit_diff"]) == 0, f"{int(r['logit_diff'])} logits differ between {world} GPUs and 1"
    assert np.array_equal(r["toks"], r["want"]), (r["toks"], r["want"])


def _run_rank_serving(rank, world, port, out_dir):
    """Three sequences with prompts of several ragged chunks advance together on a sharded model (every rank holds its
    heads' caches and states of every sequence); rank 0 also produces every stream alone on the unsharded model."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    from det_b200 import capi
    rt = C.CDLL("libcudart.so.12")
    assert rt.cudaSetDevice(rank) == 0
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    h, d = capi.host(), capi.cuda()
    backend = h.dh_cuda_backend_new(1, 1)
    assert backend, h.dh_last_error()
    nid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = np.zeros(128, np.uint8)
        h.dh_nccl_unique_id(buf.ctypes.data)
        nid = torch.from_numpy(buf)
    dist.broadcast(nid, 0)
    nid_np = nid.numpy().copy()
    chunk, ctx, n_new = 128, 1024, 6
    comm = h.dh_peer_comm_new(nid_np.ctypes.data, rank, world, 16 * max(chunk * 3072, VOCAB) + 4096)
    assert comm, h.dh_last_error()
    mine = np.zeros(64, np.uint8)
    h.dh_peer_comm_handle(comm, mine.ctypes.data)
    every = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(every, torch.from_numpy(mine))
    handles = np.concatenate([e.numpy() for e in every]).copy()
    h.dh_peer_comm_open(comm, handles.ctypes.data)
    dist.barrier()
    prompts = [700, 333, 41]            # five chunks + 60 tokens, two + 77, one ragged chunk
    sampling = (0, 1.0 / 0.7, 40, 0.95)

    def prompt(i, n):
        ids = np.zeros(n, np.int32)
        h.dh_synth_prompt(300 + i, n, VOCAB, ids.ctypes.data)
        return ids

    shard = h.dh_model_new_synth_tp(backend, b"tiny", 4, SEED, ctx, chunk, comm)
    assert shard, h.dh_last_error()
    batch = h.dh_batch_new(shard, len(prompts), ctx)
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
    assert d.det_last_error() == 0
    if rank == 0:
        full = h.dh_model_new_synth(backend, b"tiny", 4, SEED, ctx, chunk)
        assert full, h.dh_last_error()
        solo = []
        for i, n in enumerate(prompts):
            out = np.zeros(n_new, np.int32)
            cnt = C.c_size_t(0)
            assert h.dh_model_reset(full) == 0
            ids = prompt(i, n)
            assert h.dh_model_generate(full, ids.ctypes.data, n, n_new, *sampling, 7000 + i, out.ctypes.data,
                                       C.byref(cnt)) == 0, h.dh_last_error()
            assert cnt.value == n_new
            solo.append(out)
        np.savez(Path(out_dir) / "serving.npz", together=np.stack(together), solo=np.stack(solo))
    d.det_sync()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [
    2,
    # the 27B serving line's first sampled tokens differ between 1 - 2 GPUs and 4 - 8 GPUs (ranks agree with each other):
    # an unlocated defect of the sharded batched path; whether this reduced case shows it is not known
    pytest.param(4, marks=pytest.mark.xfail(strict=False, reason="open defect of the sharded batched step at 4+ GPUs")),
])
def test_sharded_serving_streams_equal_solo_streams(world, libs, tmp_path):
    """A BatchDecoder on shards against the unsharded model serving each sequence alone, sampled tokens bit for bit:
    prompts longer than a chunk (tensor-core attention behind a filled cache, ragged last chunks, NCCL chunk exchanges),
    then batched steps (row exchanges with several rows, det_attention_rows / det_gdn_rows on a shard)."""
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_run_rank_serving, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = np.load(tmp_path / "serving.npz")
    assert np.array_equal(r["together"], r["solo"]), (r["together"], r["solo"])
