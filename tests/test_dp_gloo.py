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


def _tiny_model(O, seed):
    """Two blocks of the workload's architecture at toy size, in the oracle's dict form (same on every rank)."""
    rng = np.random.default_rng(seed)
    H, HQ, HK, D, F, V, R = 256, 2, 1, 128, 256, 300, 8
    cfg = dict(n_heads=HQ, n_kv_heads=HK, head_dim=D, rms_eps=1e-6, rope_theta=1e6, vocab=V, hidden=H, ffn=F)
    shapes = dict(q=(HQ * D, H), k=(HK * D, H), v=(HK * D, H), o=(H, HQ * D), gate=(F, H), up=(F, H), down=(H, F))
    layers = []
    for l in range(2):
        P = {}
        for j, (name, (N, K)) in enumerate(shapes.items()):
            P[name] = dict(qtype=synth.TYPE_Q6_K, w=synth.make_weight(synth.TYPE_Q6_K, N, K, seed + 10 * l + j), N=N, K=K, bias=None,
                           a=(rng.standard_normal((K, R)) / np.sqrt(K)).astype(np.float32),
                           b=(rng.standard_normal((R, N)) * 0.02).astype(np.float32), rank=R, scaling=2.0)
        layers.append(dict(norm1=np.full(H, 0.4, np.float32), norm2=np.full(H, 0.4, np.float32), proj=P))
    return dict(cfg=cfg, layers=layers, embed=(O.TYPE_F16, (rng.standard_normal((V, H)) * 0.02).astype(np.float16)),
                out_norm=np.ones(H, np.float32), lm_head=(O.TYPE_F16, (rng.standard_normal((V, H)) * 0.02).astype(np.float16)))


def _rank_batch(rank, V, T=10):
    rng = np.random.default_rng(500 + rank)
    tokens = rng.integers(0, V, T).astype(np.int32)
    labels = np.roll(tokens, -1).astype(np.int32)
    labels[-1] = -100
    return tokens, labels


def _step_worker(rank, world, port, out_dir):
    """One data-parallel training step per rank on the CPU chain: own sequence -> gradients -> per-layer exchange (last
    layer first) -> clip -> AdamW.  What gt_model_forward_backward + gt_model_optimizer_step do on the GPUs."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    model = _tiny_model(O, 42)
    tokens, labels = _rank_batch(rank, model["cfg"]["vocab"])
    grads = O.new_grads(model)
    loss = O.model_forward_backward(model, tokens, labels, grads)
    flat = torch.from_numpy(O.flat_grads(model, grads).copy())
    shapes = [(n, model["layers"][0]["proj"][n]["N"], model["layers"][0]["proj"][n]["K"]) for n in dp.PROJ_ORDER]
    entries, total = dp.flat_grad_layout(shapes, 8, layers=2)
    assert total == flat.numel()
    buckets = dp.layer_buckets(entries, 2)
    assert buckets[0][0] + buckets[0][1] == total and buckets[-1][0] == 0       # last layer first, together the whole buffer
    dp.average_gradients_bucketed(flat, buckets, dist)
    g = flat.numpy()
    norm = O.clip_gradients(g, 1.0)
    off = 0
    for layer in model["layers"]:
        for name in dp.PROJ_ORDER:
            for key in ("a", "b"):
                p = layer["proj"][name][key]
                O.adamw_step(p.reshape(-1), g[off:off + p.size], np.zeros(p.size, np.float32), np.zeros(p.size, np.float32),
                             lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=1)
                off += p.size
    params = np.concatenate([layer["proj"][n][k].reshape(-1) for layer in model["layers"] for n in dp.PROJ_ORDER for k in ("a", "b")])
    np.save(os.path.join(out_dir, f"params_{rank}.npy"), params)
    np.save(os.path.join(out_dir, f"meta_{rank}.npy"), np.array([loss, norm], np.float64))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_training_step_keeps_replicas_identical(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_step_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    p0, p1 = (np.load(tmp_path / f"params_{r}.npy") for r in range(world))
    assert np.array_equal(p0, p1)                         # every rank took the same optimizer step
    m0, m1 = (np.load(tmp_path / f"meta_{r}.npy") for r in range(world))
    assert m0[1] == m1[1] and m0[0] != m1[0]              # same global norm after the exchange, different local losses
    # single process: accumulate both sequences' gradients, scale by 1/2, clip, step (LoraTrainer.cs:217-231)
    from oracle import oracle as O
    model = _tiny_model(O, 42)
    grads = O.new_grads(model)
    for r in range(world):
        O.model_forward_backward(model, *_rank_batch(r, model["cfg"]["vocab"]), grads)
    g = O.flat_grads(model, grads) * np.float32(0.5)
    norm = O.clip_gradients(g, 1.0)
    assert abs(norm - m0[1]) < 1e-5 * norm
    off = 0
    for layer in model["layers"]:
        for name in dp.PROJ_ORDER:
            for key in ("a", "b"):
                p = layer["proj"][name][key]
                O.adamw_step(p.reshape(-1), g[off:off + p.size], np.zeros(p.size, np.float32), np.zeros(p.size, np.float32),
                             lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=1)
                off += p.size
    want = np.concatenate([layer["proj"][n][k].reshape(-1) for layer in model["layers"] for n in dp.PROJ_ORDER for k in ("a", "b")])
    assert np.allclose(p0, want, rtol=1e-5, atol=1e-6)
