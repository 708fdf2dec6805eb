"""World-size-2 CPU test (gloo) of the data-parallel driver logic: buffer layout, id rendezvous, and that
sum-then-1/world over ranks equals the reference's gradient-accumulation averaging over micro-batches."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from glacier.tune_b200 import dp, synth  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    ident = dp.share_unique_id(lambda: bytes(range(128)), dist)
    assert ident == bytes(range(128))
    # every rank: one micro-batch through the reference CPU path, grads into the flat buffer
    N, K, T, R = 48, 256, 6, 16
    shapes = [("q", N, K), ("k", N // 2, K)]
    entries, total = dp.flat_grad_layout(shapes, R)
    flat = torch.zeros(total, dtype=torch.float32)
    for name, n, k in shapes:
        c = synth.make_projection_case(synth.TYPE_Q4_K, n, k, T, seed=100 + synth.PROJ_ORDINAL[name])
        rng = np.random.default_rng(1000 * rank + synth.PROJ_ORDINAL[name])        # per-rank sequence
        x = rng.standard_normal((T, k)).astype(np.float32)
        dy = rng.standard_normal((T, n)).astype(np.float32)
        _, ga, gb = O.proj_backward(synth.TYPE_Q4_K, c["w"], dy, x, k, n, T, c["a"], c["b"], R, c["scaling"], want_dx=False)
        oa, na, ob, nb = entries[(0, name)]
        flat[oa:oa + na] = torch.from_numpy(ga.reshape(-1))
        flat[ob:ob + nb] = torch.from_numpy(gb.reshape(-1))
    bucketed = flat.clone()
    dp.average_gradients_reference(flat, dist)
    # the per-bucket exchange (last projection first, as a backward pass finishes them) gives the same buffer
    dp.average_gradients_bucketed(bucketed, dp.group_buckets(entries, groups=(("k",), ("q",))), dist)
    assert torch.equal(bucketed, flat)
    np.save(os.path.join(out_dir, f"avg_{rank}.npy"), flat.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_flat_grad_layout_order_and_size():
    shapes = [(n, *synth.QWEN7B_PROJ[n]) for n in dp.PROJ_ORDER]
    entries, total = dp.flat_grad_layout(shapes, 16, layers=28)
    assert total == 40_370_176                    # trainable parameters of the 28-layer r=16 model
    assert entries[(0, "q")] == (0, 3584 * 16, 3584 * 16, 16 * 3584)
    per_layer = total // 28
    assert per_layer == 1_441_792 and entries[(1, "q")][0] == per_layer
    prev_end = 0
    for layer in range(28):
        for name in dp.PROJ_ORDER:
            oa, na, ob, nb = entries[(layer, name)]
            assert oa == prev_end and ob == oa + na
            prev_end = ob + nb


def test_group_buckets_tile_the_layer_buffer():
    """The per-group slices of the overlapped exchange are contiguous, disjoint and cover the layer's gradients."""
    from glacier.tune_b200 import dp, synth
    shapes = [(n, *synth.QWEN7B_PROJ[n]) for n in dp.PROJ_ORDER]
    entries, total = dp.flat_grad_layout(shapes, 16)
    buckets = dp.group_buckets(entries)
    assert sum(sz for _, sz in buckets) == total == 1441792
    spans = sorted(buckets)
    assert spans[0][0] == 0 and all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(len(spans) - 1))
    # backward order: the down projection's slice is the last one in the buffer and the first one sent
    assert buckets[0][0] + buckets[0][1] == total and buckets[-1][0] == 0


def test_two_rank_gradient_averaging_equals_accumulation(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    a0, a1 = (np.load(tmp_path / f"avg_{r}.npy") for r in range(world))
    assert np.array_equal(a0, a1)                 # identical replicas after the exchange
    # single-process reference: accumulate the two micro-batches, then scale by 1/2 (LoraTrainer.cs:217-220)
    from oracle import oracle as O
    N, K, T, R = 48, 256, 6, 16
    shapes = [("q", N, K), ("k", N // 2, K)]
    entries, total = dp.flat_grad_layout(shapes, R)
    acc = np.zeros(total, np.float32)
    for name, n, k in shapes:
        c = synth.make_projection_case(synth.TYPE_Q4_K, n, k, T, seed=100 + synth.PROJ_ORDINAL[name])
        ga = np.zeros((k, R), np.float32)
        gb = np.zeros((R, n), np.float32)
        for r in range(world):
            rng = np.random.default_rng(1000 * r + synth.PROJ_ORDINAL[name])
            x = rng.standard_normal((T, k)).astype(np.float32)
            dy = rng.standard_normal((T, n)).astype(np.float32)
            O.proj_backward(synth.TYPE_Q4_K, c["w"], dy, x, k, n, T, c["a"], c["b"], R, c["scaling"], ga=ga, gb=gb, want_dx=False)
        oa, na, ob, nb = entries[(0, name)]
        acc[oa:oa + na], acc[ob:ob + nb] = ga.reshape(-1), gb.reshape(-1)
    acc *= 0.5
    assert np.allclose(a0, acc, rtol=1e-5, atol=1e-6)


def _leaver(rank, world, port, out_dir):
    """Rank 1 leaves between steps (no collective in flight); rank 0 must get an error from its next exchange
    within the process-group timeout instead of waiting forever."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    flat = torch.ones(1024)
    dp.average_gradients_reference(flat, dist)          # step 1: both ranks take part
    assert torch.allclose(flat, torch.ones(1024))
    if rank == 1:
        os._exit(0)                                      # leaves without joining step 2
    outcome = "hung"
    try:
        dp.average_gradients_reference(flat, dist)      # step 2: the peer is gone
        outcome = "completed"
    except Exception as exc:  # noqa: BLE001 - any error raised by the backend is the expected outcome
        outcome = "error: " + type(exc).__name__
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_lost_rank_surfaces_as_an_error_not_a_hang(tmp_path):
    world, port = 2, _free_port()
    ctx = mp.spawn(_leaver, args=(world, port, str(tmp_path)), nprocs=world, join=False)
    import time
    deadline = time.time() + 60
    while time.time() < deadline and not (tmp_path / "outcome.txt").exists():
        time.sleep(0.2)                       # rank 1 has left; wait for rank 0's verdict (bounded)
    time.sleep(0.2)
    outcome = (tmp_path / "outcome.txt").read_text() if (tmp_path / "outcome.txt").exists() else "no outcome"
    for p in ctx.processes:
        if p.is_alive():
            p.kill()
    assert outcome.startswith("error"), outcome
