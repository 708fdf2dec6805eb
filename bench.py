#!/usr/bin/env python
"""Benchmark of the frozen-base K-quant projection path on B200.

A step is one pass of the hot path over one 512-token sequence: the seven Qwen2.5-7B layer projections
(q, k, v, o, gate, up, down; Q4_K base, LoRA r=16, alpha=32), each forward + dX + dA/dB, through
libglaciertune_b200.so.  The metric counts the base GEMM terms only: 4*M*N*K per projection, 477.28 GFLOP per
step.  With N > 1 GPUs every rank runs the same step on its own sequence (weak scaling) and the flat fp32
LoRA-gradient buffer of the layer is summed with one NCCL all-reduce inside the step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

`--impl reference` times the CPU restatement of the reference's own CPU path (the oracle) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from glacier.tune_b200 import synth  # noqa: E402

M_TOKENS = 512
RANK, ALPHA = 16, 32.0
PROJ_ORDER = ["q", "k", "v", "o", "gate", "up", "down"]
METRIC = "q4k_gemm_fwd_dx_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "qwen2.5-7b layer projections q,k,v,o,gate,up,down in Q4_K, M=512, fwd+dX+LoRA grads (r=16)"
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel, the gate,up forward
# launch (the largest of the step): a constant taken from one `ncu --set full` capture of that launch, not re-measured
# by this script.  84.5e6 read (80.1e6 algorithmic: both members' packed weights once + the bf16 activations) and
# 31.4e6 of the 77.6e6 fp32 output written back before the kernel ended (the rest was still in L2).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 115.7e6
L2_NOTE = "256 MiB written between timed steps; per-step inputs (131 MB weights + activations) exceed L2"
GROUPS = [["q", "k", "v"], ["o"], ["gate", "up"], ["down"]]


def workload_config(n_gpus: int, q4km: bool = False) -> dict:
    """The `config` object of the JSON line: the same keys and values in the GPU arm and in the reference arm."""
    return {"workload": WORKLOAD.replace("in Q4_K", "in the Q4_K_M mix (v, down in Q6_K)") if q4km else WORKLOAD,
            "tokens_per_gpu": M_TOKENS, "rank": RANK, "parallelism": f"dp{n_gpus}", "l2": L2_NOTE}


def step_flops(names=PROJ_ORDER, m=M_TOKENS) -> float:
    return float(sum(4 * m * synth.QWEN7B_PROJ[n][0] * synth.QWEN7B_PROJ[n][1] for n in names))


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(bf16_tflops=float(d["bf16_tflops"]), bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", 0)),
                    hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_layer_pass(O, cases) -> float:
    """One pass of LoraAdapter.Forward + LoraAdapter.Backward per projection on the CPU path; returns seconds."""
    t0 = time.perf_counter()
    for c in cases:
        O.proj_forward(c["qtype"], c["w"], None, c["x"], c["K"], c["N"], c["T"], c["a"], c["b"], RANK, c["scaling"])
        O.proj_backward(c["qtype"], c["w"], c["dy"], c["x"], c["K"], c["N"], c["T"], c["a"], c["b"], RANK, c["scaling"])
    return time.perf_counter() - t0


def parity_against_oracle(O, eng, layer, groups, flat_grads, q4km: bool) -> dict:
    """After the timed region: the device tensors the last step left behind (every Y, each group's dX, the flat gradient
    buffer) against the CPU path on the same seeded inputs, plus bit-equality of sampled dequantized weight rows.
    Relative Frobenius errors, worst over the projections; gate 2e-2 (bf16-MMA mode)."""
    by_name = {p["name"]: p for p in layer}
    worst = {"Y": 0.0, "dX": 0.0, "dA": 0.0, "dB": 0.0}
    bit_exact = True
    grads = flat_grads.cpu().numpy()
    for names in groups:
        ps = [by_name[n] for n in names]
        x = ps[0]["hx"].numpy()                       # the group's shared input
        K = ps[0]["K"]
        dx_ref = np.zeros((M_TOKENS, K), np.float32)
        for p in ps:
            c = p["case"]
            y_ref = O.proj_forward(c["qtype"], c["w"], None, x, K, p["N"], M_TOKENS, c["a"], c["b"], RANK, c["scaling"])
            _, da_ref, db_ref = O.proj_backward(c["qtype"], c["w"], c["dy"], x, K, p["N"], M_TOKENS, c["a"], c["b"], RANK,
                                                c["scaling"], dx=dx_ref)
            worst["Y"] = max(worst["Y"], O.rel_fro(p["Y"].cpu().numpy(), y_ref))
            g0 = p["g0"]
            da = grads[g0: g0 + K * RANK].reshape(K, RANK)
            db = grads[g0 + K * RANK: g0 + K * RANK + RANK * p["N"]].reshape(RANK, p["N"])
            worst["dA"] = max(worst["dA"], O.rel_fro(da, da_ref))
            worst["dB"] = max(worst["dB"], O.rel_fro(db, db_ref))
            rows = [0, p["N"] // 2 + 1, p["N"] - 1]
            for r in rows:
                got = eng.dequant_rows(p["w"], r, 1)
                want = O.dequant_rows(c["qtype"], c["w"], K, r, 1)
                bit_exact = bit_exact and bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
        worst["dX"] = max(worst["dX"], O.rel_fro(ps[0]["dX"].cpu().numpy(), dx_ref))
    out = {k: float(v) for k, v in worst.items()}
    out["dequant_bit_exact"] = bit_exact
    out["gate"] = 2e-2
    out["ok"] = bool(bit_exact and all(v < 2e-2 for v in worst.values()))
    out["checked"] = ("all seven projections of the last timed step (Y, group dX, dA, dB) against the CPU path, fp32; "
                      "three dequantized rows per weight bit for bit" + ("; Q4_K_M mix" if q4km else ""))
    return out


def make_cpu_cases(names, seed_base=0):
    return [synth.make_projection_case(synth.TYPE_Q4_K, *synth.QWEN7B_PROJ[n], M_TOKENS,
                                       synth.seed_for(1, 0, n) + seed_base, rank=RANK, alpha=ALPHA, x_bf16=True)
            for n in names]


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    O.set_threads(os.cpu_count() or 1)           # torchrun pins OMP_NUM_THREADS=1; the CPU arm uses every host core
    cores = O.num_threads()
    budget_s = 150.0
    names = list(PROJ_ORDER)
    cases = make_cpu_cases(["k"])
    cpu_layer_pass(O, cases)                      # page in / warm the thread pool
    probe = make_cpu_cases(["q"])
    t_q = cpu_layer_pass(O, probe)
    est_full = t_q * step_flops() / step_flops(["q"])
    if est_full * (args.steps + args.warmup) > budget_s:
        names = ["q", "k", "v", "o"]
        if t_q * step_flops(names) / step_flops(["q"]) * (args.steps + args.warmup) > budget_s:
            names = ["q"]
    cases = make_cpu_cases(names)
    for _ in range(args.warmup):
        cpu_layer_pass(O, cases)
    times = [cpu_layer_pass(O, cases) for _ in range(args.steps)]
    total = sum(times)
    fl = step_flops(names)
    value = fl * args.steps / total / 1e12
    sample = f"projections {','.join(names)} of the workload per step ({fl / 1e9:.1f} GFLOP), fp32, OpenMP"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms from the warm-up to the end of the timed region
    (samples below 250 W are idle and dropped)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.NamedTemporaryFile(prefix="gt_clocks_", suffix=".csv", delete=False).name
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                          "50", "-i", str(self.gpu_index)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for ln in f:
                    p = [x.strip() for x in ln.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        if float(p[3]) < 250.0:       # idle samples (before the load starts) are not "under load"
                            continue
                        sm.append(float(p[1]))
                        mx.append(float(p[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def _log(msg: str) -> None:
    if os.environ.get("GT_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from glacier.tune_b200 import capi as G

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries exactly one JSON line: anything a library prints there meanwhile (NCCL's version banner) is sent
    # to stderr, and the line itself is written to the saved descriptor
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(text: str) -> None:
        os.write(real_stdout, (text + "\n").encode())

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the projection path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"          # the version banner goes to stdout, which carries the JSON line
        dist.init_process_group("nccl", device_id=dev)

    # a real (non-default) stream shared by torch and the engine, so torch.cuda.Event brackets the engine's kernels
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    eng = G.Engine(local_rank, G.MATH_BF16, stream=stream.cuda_stream)

    # ---- build the layer: weights, adapters (grads bound into one flat buffer in the reference's order)
    n_grad = sum(RANK * (synth.QWEN7B_PROJ[n][0] + synth.QWEN7B_PROJ[n][1]) for n in PROJ_ORDER)
    flat_grads = torch.zeros(n_grad, dtype=torch.float32, device=dev)
    layer, off = [], 0
    for n in PROJ_ORDER:
        N, K = synth.QWEN7B_PROJ[n]
        qt = synth.TYPE_Q6_K if (args.q4km and n in ("v", "down")) else synth.TYPE_Q4_K
        c = synth.make_projection_case(qt, N, K, M_TOKENS, synth.seed_for(2 if args.q4km else 1, 0, n) + 100000 * rank, rank=RANK,
                                       alpha=ALPHA, x_bf16=True)
        w = eng.upload_weight(qt, c["w"], N, K)
        ad = eng.create_adapter(K, N, RANK, ALPHA)
        ad.upload(c["a"], c["b"])
        g0 = off
        dA = flat_grads[off: off + K * RANK]; off += K * RANK
        dB = flat_grads[off: off + RANK * N]; off += RANK * N
        ad.bind_grads(dA, dB)
        pin = lambda a: torch.from_numpy(a).pin_memory()   # noqa: E731
        hx, hdy = pin(c["x"]), pin(c["dy"])
        layer.append(dict(name=n, N=N, K=K, w=w, ad=ad, hx=hx, hdy=hdy, g0=g0, g1=off, case=c if rank == 0 else None,
                          hy=torch.empty((M_TOKENS, N), dtype=torch.float32).pin_memory(),
                          hdx=torch.zeros((M_TOKENS, K), dtype=torch.float32).pin_memory(),
                          X=hx.to(dev), dY=hdy.to(dev), Y=torch.empty((M_TOKENS, N), dtype=torch.float32, device=dev),
                          dX=torch.empty((M_TOKENS, K), dtype=torch.float32, device=dev)))
    if world > 1:
        ident = [eng.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
        eng.dp_init(world, rank, ident[0])

    _log("layer built")
    l2_flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    # q,k,v read the same normed hidden state and gate,up the same FFN input (TransformerBlock.Forward): each group is
    # one call that shares the input and sums the members' input gradients into one buffer
    by_name = {p["name"]: p for p in layer}
    groups = GROUPS if not args.no_group else [[n] for n in PROJ_ORDER]
    calls = []
    for names in groups:
        ps = [by_name[n] for n in names]
        calls.append(dict(ws=[p["w"] for p in ps], ads=[p["ad"] for p in ps], X=ps[0]["X"], Ys=[p["Y"] for p in ps],
                          dYs=[p["dY"] for p in ps], dX=ps[0]["dX"],
                          grads=flat_grads[ps[0]["g0"]: ps[-1]["g1"]]))      # the group's slice of the flat gradient buffer

    def step_resident(exchange: bool = True):
        flat_grads.zero_()
        for c in calls:
            if len(c["ws"]) > 1:
                eng.forward_group(c["ws"], c["ads"], c["X"], c["Ys"])
            else:
                eng.forward(c["ws"][0], c["ads"][0], c["X"], c["Ys"][0])
        # X is the tensor the forward above saw: X*A kept by the adapter is reused (GT_FLAG_REUSE_LOW).  The reference
        # hands Backward a zero-filled dX (AutogradScratchWorkspace.Wrap) and accumulates; GT_FLAG_DX_ASSIGN makes
        # the call clear dX itself ("dX ="), --zero-dx keeps the separate fill and the "+=" call
        bflags = G.FLAG_REUSE_LOW | (0 if args.zero_dx else G.FLAG_DX_ASSIGN)
        for c in reversed(calls):
            if args.zero_dx:
                c["dX"].zero_()
            if len(c["ws"]) > 1:
                eng.backward_group(c["ws"], c["ads"], c["dYs"], c["X"], c["dX"], flags=bflags)
            else:
                eng.backward(c["ws"][0], c["ads"][0], c["dYs"][0], c["X"], c["dX"], flags=bflags)
            # the group's gradients are final: their all-reduce runs beside the backward of the groups that follow
            if world > 1 and args.overlap and exchange:
                eng.dp_allreduce_begin(c["grads"], 1.0 / world)
        if world > 1 and args.overlap and exchange:
            eng.dp_allreduce_end()
        if world > 1 and not args.overlap and exchange:
            eng.dp_allreduce(flat_grads, 1.0 / world)

    # end to end: the same grouped calls on page-locked HOST buffers.  Every call stages its inputs to the device and its
    # results back; GT_FLAG_HOST_ASYNC queues them (uploads, kernels and downloads of consecutive calls overlap) and
    # gt_sync() completes the step, after which every Y and dX is in host memory.
    hcalls = []
    for names in groups:
        ps = [by_name[n] for n in names]
        hcalls.append(dict(ws=[p["w"] for p in ps], ads=[p["ad"] for p in ps], X=ps[0]["hx"].numpy(),
                           Ys=[p["hy"].numpy() for p in ps], dYs=[p["hdy"].numpy() for p in ps], dX=ps[0]["hdx"].numpy()))
    hflags = 0 if args.e2e_sync else G.FLAG_HOST_ASYNC
    # with GT_FLAG_REUSE_LOW the backward reuses the device copy of X that the forward staged: X goes up once
    e2e_h2d = sum(c["X"].nbytes + sum(d.nbytes for d in c["dYs"]) for c in hcalls)
    e2e_d2h = sum(sum(y.nbytes for y in c["Ys"]) + c["dX"].nbytes for c in hcalls)

    def step_host():
        for c in hcalls:
            eng.forward_group(c["ws"], c["ads"], c["X"], c["Ys"], flags=hflags)
        for c in reversed(hcalls):
            eng.backward_group(c["ws"], c["ads"], c["dYs"], c["X"], c["dX"], flags=hflags | G.FLAG_DX_ASSIGN | G.FLAG_REUSE_LOW)
        if world > 1:
            eng.dp_allreduce(flat_grads, 1.0 / world)
        eng.sync()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing.  The clock sampler starts before the warm-up, and the warm-up runs for at
    # least half a second so that the clocks have ramped and nvidia-smi has samples taken under load.
    if args.launch_list and args.workload == "step":
        # the training step of a few layers for a profiler's launch list (the LM head stays full size)
        import torch as _t
        # (one launch per kernel: a profiler lists the kernels of a graph replay less readably)
        model, keep, heads, _ = build_step_model(G, eng, dev, args.train_layers, rank, M_TOKENS, graph=False)
        rng_ = np.random.default_rng(4000)
        tok = rng_.integers(0, STEP_CFG["vocab"], M_TOKENS).astype(np.int32)
        lab = np.roll(tok, -1).astype(np.int32)
        lab[-1] = -100
        tok_d, lab_d = _t.from_numpy(tok).to(dev), _t.from_numpy(lab).to(dev)
        loss_d = _t.zeros(1, device=dev)
        for i in range(args.warmup + args.steps):
            model.forward_backward(tok_d, lab_d, loss_dev=loss_d)
            model.optimizer_step(step=i + 1, max_norm=1.0, **ADAMW)
        eng.sync()
        emit(json.dumps({"launch_list": True, "workload": "step", "layers": args.train_layers, "steps": args.steps, "warmup": args.warmup,
                         "loss": float(loss_d.item())}))
        model.close()
        eng.close()
        return
    if args.launch_list:
        # a short eager run for a profiler's launch list: W warm-up steps, K steps, no timing, no other legs
        for _ in range(args.warmup + args.steps):
            l2_flush.zero_()
            step_resident()
        eng.sync()
        emit(json.dumps({"launch_list": True, "steps": args.steps, "warmup": args.warmup, "config": workload_config(world, args.q4km)}))
        eng.close()
        return
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    warm_t0, n_warm = time.perf_counter(), 0
    while True:
        # every rank must run the same number of steps (each holds an all-reduce): warm up in chunks and let the
        # ranks agree on whether another chunk is needed
        for _ in range(max(args.warmup, 3) if n_warm == 0 else 50):
            step_resident()
            l2_flush.zero_()
            n_warm += 1
        torch.cuda.synchronize()
        more = torch.tensor([1 if time.perf_counter() - warm_t0 < 0.6 else 0], dtype=torch.int32, device=dev)
        if world > 1:
            dist.all_reduce(more, op=dist.ReduceOp.MAX)
        if int(more.item()) == 0:
            break
    _log(f"warm-up done ({n_warm} steps)")
    eng.sync()
    # The step is launch-bound on the host side (about 55 short kernels): capture it once in a CUDA graph and time
    # replays.  The engine enqueues on the stream torch captures; nothing in the step allocates after the warm-up.
    graph = None
    if not args.no_graph:
        try:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                step_resident()
            torch.cuda.set_stream(stream)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001 - fall back to eager launches, and say so in the output
            print(f"bench.py: CUDA graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            graph = None
            torch.cuda.set_stream(stream)
            torch.cuda.synchronize()
    run_step = graph.replay if graph is not None else step_resident
    _log(f"graph={'yes' if graph is not None else 'no'}")
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        l2_flush.zero_()                      # > L2 (126 MB) written between timed steps
        starts[i].record(stream)
        run_step()
        ends[i].record(stream)
    barrier()
    # A second, long measurement of the same step for the clock record: the K timed steps above last a few
    # milliseconds, less than one nvidia-smi sample, so the sampler mostly sees the warm-up.  `sustained_steps` steps
    # (about half a second) between event pairs per step, L2 flushed as above; reported beside the headline with
    # time x median SM clock.
    sus_n = max(args.steps, int(args.sustained_steps))
    sus_a = [torch.cuda.Event(enable_timing=True) for _ in range(sus_n)]
    sus_b = [torch.cuda.Event(enable_timing=True) for _ in range(sus_n)]
    for i in range(sus_n):
        l2_flush.zero_()
        sus_a[i].record(stream)
        run_step()
        sus_b[i].record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else {}
    eng.sync()
    sus_ms = sum(a.elapsed_time(b) for a, b in zip(sus_a, sus_b))
    # Per-kernel numbers for the roofline: the same steps once more with eager launches, every tensor-core GEMM
    # bracketed by CUDA events on the launching stream, L2 flushed between steps as above.
    eng.profile_read(reset=True)
    eng.profile_enable(True)
    prof_steps = min(args.steps, 10)
    for _ in range(prof_steps):
        l2_flush.zero_()
        step_resident()
    eng.sync()
    prof = eng.profile_read(reset=True)
    eng.profile_enable(False)
    launches_per_step = prof["kernel_launches"] // max(1, prof_steps)
    total_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
    t = torch.tensor([total_ms, sus_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, sus_ms = float(t[0].item()), float(t[1].item())
    fl = step_flops()
    value = world * fl * args.steps / (total_ms * 1e-3) / 1e12

    _log("timed region done")
    # ---- parity of what the timed steps computed (rank 0): the device tensors of the last step against the CPU path
    parity = None
    if rank == 0 and not args.no_parity:
        from oracle import oracle as O
        O.build()
        O.set_threads(os.cpu_count() or 1)       # torchrun pins OMP_NUM_THREADS=1
        step_resident(exchange=False)            # one eager step of this rank alone: its outputs are what is compared
        eng.sync()
        parity = parity_against_oracle(O, eng, layer, groups, flat_grads, args.q4km)
        _log(f"parity {parity}")
    barrier()
    # ---- end to end through the C ABI with host buffers (H2D of the inputs, D2H of the results, every step)
    e2e_steps = max(1, int(args.e2e_steps))
    for _ in range(5):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_host()
    barrier()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    e2e_value = world * fl * e2e_steps / e2e_s / 1e12
    h2d, d2h = e2e_h2d, e2e_d2h     # per group: X (forward) and every dY (backward) up; every Y and one dX down

    _log("e2e done")
    # ---- the 28-layer training step (tokens/s): every rank takes part (per-block gradient exchange at N > 1)
    train = None
    if not args.no_train_step:
        def _max(v):
            t_ = torch.tensor([float(v)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            return float(t_.item())
        try:
            train = run_train_step(G, eng, dev, stream, world, rank, args.train_steps, 3, args.train_layers, barrier, _max)
        except Exception as exc:  # noqa: BLE001 - the headline line must still print; the failure is reported in it
            train = {"error": f"{type(exc).__name__}: {exc}"}
        _log(f"train step {train}")
    if rank == 0:
        peaks = measured_peaks()
        gemm_tflops = prof["gemm_flops"] / (prof["gemm_ms"] * 1e-3) / 1e12 if prof["gemm_ms"] > 0 else 0.0
        roofline = {
            "bound": "tensor", "kernel": "k_umma_gemm (tcgen05 Q4_K forward / dX)",
            "achieved": gemm_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": gemm_tflops / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} burst bf16",
            "frac_of_sustained": (gemm_tflops / peaks["bf16_tflops_sustained"]) if peaks["bf16_tflops_sustained"] else None,
            "timed_in": f"eager pass of {prof_steps} steps after the timed region (events around each GEMM launch)",
            "launches": prof["gemm_launches"], "avg_launch_us": 1e3 * prof["gemm_ms"] / max(1, prof["gemm_launches"]),
            "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
            "traffic_source": "constant from one ncu --set full capture of this launch (dram__bytes_read.sum + dram__bytes_write.sum); not re-measured by this run",
            "traffic_of": "gate,up forward launch, 2 x 18944x3584 at M=512 (algorithmic HBM bytes: 80.1e6 read + 77.6e6 fp32 output, of which 31.1e6 left the L2 before the kernel ended)",
        }
        # CPU baseline: the oracle (a port of the reference's CPU path) on this host, one pass over the same layer
        from oracle import oracle as O
        O.build()
        O.set_threads(os.cpu_count() or 1)       # torchrun pins OMP_NUM_THREADS=1
        cpu_layer_pass(O, make_cpu_cases(["k"]))
        names = list(PROJ_ORDER)
        t_q = cpu_layer_pass(O, make_cpu_cases(["q"]))
        if t_q * step_flops() / step_flops(["q"]) > 45.0:
            names = ["q", "k", "v", "o"]
        cpu_s = cpu_layer_pass(O, make_cpu_cases(names))
        cpu_val = step_flops(names) / cpu_s / 1e12
        ms_step = total_ms / args.steps
        sus_ms_step = sus_ms / sus_n
        sm_mhz = clocks.get("sm_mhz") if isinstance(clocks, dict) else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, args.q4km),
            "detail": {"launch": "cuda graph replay" if graph is not None else "eager", "warmup_run": n_warm,
                       "tokens_per_s_through_one_layer": world * M_TOKENS * args.steps / (total_ms * 1e-3),
                       "sustained": {"steps": sus_n, "ms_per_step": sus_ms_step,
                                     "value": world * fl / (sus_ms_step * 1e-3) / 1e12,
                                     "ms_x_sm_mhz": (sus_ms_step * sm_mhz) if sm_mhz else None},
                       "ms_x_sm_mhz": (ms_step * sm_mhz) if sm_mhz else None},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "warmup": 5, "ms_per_step": 1e3 * e2e_s / e2e_steps,
                    "calls": "grouped host-buffer calls, " + ("synchronous" if args.e2e_sync else "queued (GT_FLAG_HOST_ASYNC) + gt_sync per step")},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": roofline,
            "cpu_baseline": {"value": cpu_val, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                             "sample": f"one pass over projections {','.join(names)} ({step_flops(names) / 1e9:.1f} GFLOP), fp32 OpenMP"},
            "parity": parity,
            "train_step": train,
            "clocks": clocks,
        }
        emit(json.dumps(line))
    if graph is not None:
        graph.reset()          # a communicator cannot be torn down while a captured graph still references it
        graph = None
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        eng.dp_finalize()
        dist.destroy_process_group()
    eng.close()



# ------------------------------------------------------------------------------------------------ 28-layer training step
STEP_WORKLOAD = ("qwen2.5-7b-architecture LoRA training step: 28 layers, hidden 3584, 28/4 heads x 128, FFN 18944, vocab 152064, "
                 "Q4_K_M-mixed base (v, down in Q6_K), fp16 embedding and LM head, r=16 on q,k,v,o,gate,up,down, one 512-token "
                 "sequence per GPU, activation checkpointing (block inputs kept; each block's state is recomputed before its "
                 "backward, up to but not including the down projection, whose output is the next block's kept input), "
                 "streaming cross-entropy, clip 1.0, AdamW lr 2e-4")
STEP_CFG = dict(n_layers=28, hidden=3584, n_heads=28, n_kv_heads=4, head_dim=128, ffn=18944, vocab=152064)
ADAMW = dict(lr=2e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


def step_projection_flops(n_layers: int, checkpoint: bool = True) -> float:
    """Base-term FLOPs of the projections in one step: forward (twice with checkpoint recompute) + dX."""
    per_layer_fwd = step_flops() / 2.0
    return n_layers * per_layer_fwd * (3.0 if checkpoint else 2.0)


def build_step_model(G, eng, dev, n_layers: int, rank: int, max_tokens: int, checkpoint: bool = True, reuse=None, graph: bool = True):
    """The config-3 model on the device: seeded synthetic weights (one layer's K-quant bytes drawn on the host, the other
    layers' quant fields derived from them by a seeded XOR - scales and mins shared), A ~ N(0, 1/sqrt(in)), B = 0."""
    import torch
    c = STEP_CFG
    m = G.Model(eng, n_layers, c["hidden"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["ffn"], c["vocab"], max_tokens,
                rms_eps=1e-6, rope_theta=1e6, checkpoint=checkpoint, graph=graph)
    if reuse is not None:      # a second model over the same weight and adapter handles (e.g. without checkpointing)
        keep, heads = reuse
        ones = np.ones(c["hidden"], np.float32)
        for l, (ws, ads) in enumerate(keep):
            m.set_block(l, ws, ads, ones, ones)
        m.set_head(heads[0], ones, heads[1])
        _, n_grads = m.bind_grads()
        return m, keep, heads, n_grads
    base = {}
    for n in PROJ_ORDER:
        N, K = synth.QWEN7B_PROJ[n]
        qt = synth.TYPE_Q6_K if n in ("v", "down") else synth.TYPE_Q4_K
        base[n] = (qt, N, K, synth.make_weight(qt, N, K, synth.seed_for(3, 0, n)))
    keep = []
    rng = np.random.default_rng(3000 + rank)
    ones = np.ones(c["hidden"], np.float32)
    for l in range(n_layers):
        ws, ads = [], []
        for n in PROJ_ORDER:
            qt, N, K, w0 = base[n]
            w = w0
            if l > 0:
                bb = 144 if qt == synth.TYPE_Q4_K else 210
                blocks = w0.reshape(-1, bb).copy()
                lo, hi = (16, 144) if qt == synth.TYPE_Q4_K else (0, 192)       # the quant bytes of a block
                mask = np.random.default_rng(7919 * l + synth.PROJ_ORDINAL[n]).integers(0, 256, hi - lo, dtype=np.uint8)
                blocks[:, lo:hi] ^= mask
                w = blocks.reshape(-1)
            bias = np.zeros(N, np.float32) if n in ("q", "k", "v") else None      # qwen2 carries q/k/v biases (zero here)
            ws.append(eng.upload_weight(qt, w, N, K, bias))
            ad = eng.create_adapter(K, N, RANK, ALPHA)
            ad.upload((rng.standard_normal((K, RANK)) / np.sqrt(K)).astype(np.float32), np.zeros((RANK, N), np.float32))
            ads.append(ad)
        m.set_block(l, ws, ads, ones, ones)
        keep.append((ws, ads))
    heads = []
    for seed in (11, 12):
        g = torch.Generator(device=dev)
        g.manual_seed(seed + 100 * rank)
        t = (torch.randn((c["vocab"], c["hidden"]), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.float16)
        heads.append(eng.upload_weight(G.TYPE_F16, t.cpu().numpy(), c["vocab"], c["hidden"]))
        del t
    m.set_head(heads[0], ones, heads[1])
    _, n_grads = m.bind_grads()
    torch.cuda.empty_cache()
    return m, keep, heads, n_grads


def run_train_step(G, eng, dev, stream, world: int, rank: int, steps: int, warmup: int, n_layers: int, barrier, allreduce_max) -> dict:
    """The full training step on this rank's own sequence; with a communicator on the engine every block's gradients
    are averaged over the ranks beside the backward of the blocks below.  Returns the measurements (rank 0 prints)."""
    import torch
    T = M_TOKENS
    t_build = time.perf_counter()
    model, keep, heads, n_grads = build_step_model(G, eng, dev, n_layers, rank, T)
    build_s = time.perf_counter() - t_build
    rng = np.random.default_rng(4000 + rank)
    tokens = rng.integers(0, STEP_CFG["vocab"], T).astype(np.int32)
    labels = np.roll(tokens, -1).astype(np.int32)
    labels[-1] = -100
    tok_d, lab_d = torch.from_numpy(tokens).to(dev), torch.from_numpy(labels).to(dev)
    total = warmup + steps
    losses = torch.zeros(total + 1, dtype=torch.float32, device=dev)

    def one_step(i):
        model.forward_backward(tok_d, lab_d, loss_dev=losses[i:i + 1])
        model.optimizer_step(step=i + 1, max_norm=1.0, **ADAMW)

    for i in range(warmup):
        one_step(i)
    eng.sync()
    barrier()
    a = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    b = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        a[i].record(stream)
        one_step(warmup + i)
        b[i].record(stream)
    barrier()
    eng.sync()
    ms = allreduce_max(sum(x.elapsed_time(y) for x, y in zip(a, b)))
    graph_info = model.step_info()      # the timed steps were replays of the captured step (all but the first two calls)
    # share of the tensor-core GEMMs (projections and LM head), one eager step with events around each launch
    eng.profile_read(reset=True)
    eng.profile_enable(True)
    model.forward_backward(tok_d, lab_d, loss_dev=losses[total:total + 1])
    eng.sync()
    prof = eng.profile_read(reset=True)
    eng.profile_enable(False)
    model.optimizer_step(step=total + 1, max_norm=1.0, **ADAMW)
    # end to end: host token ids in, loss back on the host, every step
    barrier()
    e2e_n = max(2, min(steps, 5))
    t0 = time.perf_counter()
    host_losses = []
    for i in range(e2e_n):
        host_losses.append(model.forward_backward(tokens, labels))
        model.optimizer_step(step=total + 2 + i, max_norm=1.0, **ADAMW)
    eng.sync()
    barrier()
    e2e_s = allreduce_max(time.perf_counter() - t0)
    ls = [float(v) for v in losses.cpu().numpy()[:total]]
    ms_step = ms / steps
    # the same step WITHOUT activation checkpointing (not the workload's configuration; reported beside it): 180 GB of HBM
    # hold every block's state (4.3 GB at 512 tokens), so the recomputed forward - a third of the projection work - goes
    no_ckpt = None
    try:
        model.close()
        model = None
        m2, _, _, _ = build_step_model(G, eng, dev, n_layers, rank, T, checkpoint=False, reuse=(keep, heads))
        for i in range(3):
            m2.forward_backward(tok_d, lab_d, loss_dev=losses[total:total + 1])
            m2.optimizer_step(step=99 + i, max_norm=1.0, **ADAMW)
        eng.sync()
        barrier()
        n2 = max(3, steps // 2)
        a2 = [torch.cuda.Event(enable_timing=True) for _ in range(n2)]
        b2 = [torch.cuda.Event(enable_timing=True) for _ in range(n2)]
        for i in range(n2):
            a2[i].record(stream)
            m2.forward_backward(tok_d, lab_d, loss_dev=losses[total:total + 1])
            m2.optimizer_step(step=102 + i, max_norm=1.0, **ADAMW)
            b2[i].record(stream)
        barrier()
        eng.sync()
        ms2 = allreduce_max(sum(x.elapsed_time(y) for x, y in zip(a2, b2))) / n2
        no_ckpt = {"ms_per_step": ms2, "tokens_per_s": world * T * 1e3 / ms2, "steps": n2,
                   "note": "activation checkpointing off: every block's state kept in HBM, no recomputed forward"}
        m2.close()
    except Exception as exc:  # noqa: BLE001
        no_ckpt = {"error": f"{type(exc).__name__}: {exc}"}
    out = {
        "workload": STEP_WORKLOAD if n_layers == 28 else STEP_WORKLOAD.replace("28 layers", f"{n_layers} layers"),
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
        "tokens_per_s": world * T * 1e3 / ms_step,
        "projection_tflops": world * step_projection_flops(n_layers) / (ms_step * 1e-3) / 1e12,
        "gemm_ms_per_step": prof["gemm_ms"], "gemm_launches_per_step": prof["gemm_launches"],
        "gemm_tflops": prof["gemm_flops"] / (prof["gemm_ms"] * 1e-3) / 1e12 if prof["gemm_ms"] > 0 else 0.0,
        "kernel_launches_per_step": prof["kernel_launches"],
        "cuda_graph": {"timed_steps_replayed": bool(graph_info["graph_ready"] and graph_info["replays"] >= steps),
                       "kernels_per_replay": graph_info["kernels_per_replay"]},
        "lora_parameters": n_grads, "gradient_exchange": ("per-block ncclAllReduce(avg) on a side stream, last block first" if world > 1 else "none"),
        "loss_first_steps": ls[:10], "loss_finite": bool(np.all(np.isfinite(ls))),
        "e2e": {"tokens_per_s": world * T * e2e_n / e2e_s, "ms_per_step": 1e3 * e2e_s / e2e_n, "steps": e2e_n,
                "h2d_bytes_per_step": 2 * T * 4, "d2h_bytes_per_step": 12, "loss": host_losses[-1]},
        "without_checkpointing": no_ckpt,
        "build_s": build_s,
    }
    if model is not None:
        model.close()
    for ws, ads in keep:
        for h in ws + ads:
            h.free()
    for h in heads:
        h.free()
    return out

# ------------------------------------------------------------------------------------------------ M sweep
def run_sweep(args) -> None:
    """Token-count sweep of the Q4_K_M-mixed 7B projection set (v and down in Q6_K): device time of one projection
    call, forward and dX, per projection and M, against the roofline that bounds it (weight streaming from HBM for few
    tokens, the tensor pipe for many).  Prints one JSON line {"sweep": [...]}; a table goes to stderr."""
    import torch
    from glacier.tune_b200 import capi as G
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --sweep: no CUDA device")
    peaks = measured_peaks()
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    eng = G.Engine(0, G.MATH_BF16, stream=stream.cuda_stream)
    rows = []
    L2_BYTES = 126 << 20
    for name in ("q", "k", "v", "gate", "down"):
        N, K = synth.QWEN7B_PROJ[name]
        qt = synth.TYPE_Q6_K if name in ("v", "down") else synth.TYPE_Q4_K
        c = synth.make_projection_case(qt, N, K, 1, synth.seed_for(2, 0, name))
        wbytes = N * K // 256 * (144 if qt == synth.TYPE_Q4_K else 210)       # GGUF bytes: the algorithmic weight traffic
        # copies of the tensor that the timed calls walk round-robin: together larger than L2, so every call streams its
        # weights from HBM without a flush kernel between the calls
        copies = max(2, min(32, -(-(192 << 20) // wbytes)))
        ws = [eng.upload_weight(qt, c["w"], N, K) for _ in range(copies)]
        for M in args.sweep_m:
            X = torch.randn((M, K), device="cuda")
            dY = torch.randn((M, N), device="cuda")
            Y = torch.empty((M, N), device="cuda")
            dX = torch.zeros((M, K), device="cuda")
            for direction in ("fwd", "dx"):
                def one(w):
                    if direction == "fwd":
                        eng.forward(w, None, X, Y)
                    else:
                        eng.backward(w, None, dY, None, dX)
                for w in ws:
                    one(w)
                eng.sync()
                # one pass over the copies, captured once and replayed: a call at a handful of tokens is shorter than the
                # host time to issue it
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                    for w in ws:
                        one(w)
                graph.replay()
                passes = 3
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record(stream)
                for _ in range(passes):
                    graph.replay()
                e1.record(stream)
                e1.synchronize()
                us = 1e3 * e0.elapsed_time(e1) / (passes * copies)
                graph.reset()
                # the GEMM launch alone (the engine's events around it; each event pair costs a few microseconds, which
                # shows at few tokens): the figure to hold against the tensor roofline at many tokens, where the call also
                # spends time casting its activations
                eng.profile_read(True)
                eng.profile_enable(True)
                for w in ws[:4]:
                    one(w)
                pr = eng.profile_read(True)
                eng.profile_enable(False)
                kernel_us = 1e3 * pr["gemm_ms"] / max(1, pr["gemm_launches"])
                tf = 2.0 * M * N * K / us / 1e6
                gbs = wbytes / us / 1e3
                rows.append({"proj": name, "qtype": "Q6_K" if qt == synth.TYPE_Q6_K else "Q4_K", "N": N, "K": K, "M": M,
                             "dir": direction, "us": us, "tflops": tf, "frac_tensor": tf / peaks["bf16_tflops"],
                             "weight_gbs": gbs, "frac_hbm": gbs / peaks["hbm_gbs"], "copies": copies,
                             "l2_resident": copies * wbytes < L2_BYTES, "kernel_us": kernel_us,
                             "kernel_tflops": 2.0 * M * N * K / kernel_us / 1e6})
                print(f"{name:5s} {rows[-1]['qtype']} M={M:5d} {direction:3s}: {us:8.1f} us {tf:8.1f} TFLOP/s ({100 * tf / peaks['bf16_tflops']:5.1f} % of "
                      f"{peaks['bf16_tflops']:.0f})  weights {gbs:7.1f} GB/s ({100 * gbs / peaks['hbm_gbs']:5.1f} % of {peaks['hbm_gbs']:.0f})"
                      f"  kernel {kernel_us:7.1f} us{'  [weights fit L2]' if rows[-1]['l2_resident'] else ''}", file=sys.stderr, flush=True)
        for w in ws:
            w.free()
    eng.close()
    print(json.dumps({"sweep": rows, "peaks": peaks,
                      "timing": "whole projection call (16-bit cast of the activations, output fill where split-K adds into it, GEMM "
                                "kernel), device pointers, no adapter: CUDA events around 3 passes over `copies` copies of the weight "
                                "tensor called back to back (together larger than the 126 MB L2 unless marked l2_resident), replayed from a CUDA "
                                "graph, time per call; kernel_us = the engine's CUDA events around the GEMM launch alone, mean of 4 calls"}),
          flush=True)


# ------------------------------------------------------------------------------------------------ layer glue
def run_glue(args) -> None:
    """HBM throughput of the layer-glue kernels at the 7B layer's shapes (M = 512): algorithmic bytes / device time,
    against the measured copy bandwidth.  One JSON line {"glue": [...]}; a table goes to stderr."""
    import torch
    from glacier.tune_b200 import capi as G
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --glue: no CUDA device")
    peaks = measured_peaks()
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    eng = G.Engine(0, G.MATH_BF16, stream=stream.cuda_stream)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    T, H, F, HQ, HK, D = M_TOKENS, 3584, 18944, 28, 4, 128
    t = lambda *shape: torch.randn(shape, device="cuda")        # noqa: E731
    gate, up, dh, hid, dg, du = t(T, F), t(T, F), t(T, F), t(T, F), t(T, F), t(T, F)
    x, w, y, dy, dx = t(T, H), torch.ones(H, device="cuda"), t(T, H), t(T, H), t(T, H)
    q, k = t(T, HQ * D), t(T, HK * D)
    NP = 40_370_176
    ap_, ag_, am_, av_ = t(NP), t(NP), torch.zeros(NP, device="cuda"), torch.zeros(NP, device="cuda")
    cases = [
        ("swiglu_forward [512, 18944]", lambda: eng.swiglu_forward(gate, up, hid), 3 * 4 * T * F),
        ("swiglu_backward [512, 18944]", lambda: eng.swiglu_backward(dh, gate, up, dg, du), 5 * 4 * T * F),
        ("rmsnorm_forward [512, 3584]", lambda: eng.rmsnorm_forward(x, w, y), 2 * 4 * T * H),
        ("rmsnorm_backward [512, 3584]", lambda: eng.rmsnorm_backward(dy, x, w, dx), 3 * 4 * T * H),
        ("rope q 28 + k 4 heads x 128", lambda: eng.rope(q, k, T, HQ, HK, D, 1e6), 2 * 4 * T * (HQ + HK) * D),
        ("add [512, 3584]", lambda: eng.add(x, y, dx), 3 * 4 * T * H),
        # all adapters of the 28-layer model as one flat buffer: p, g, m, v read, p, m, v written
        ("adamw_step 40.4 M parameters", lambda: eng.adamw_step(ap_, ag_, am_, av_, 2e-4, 0.9, 0.999, 1e-8, 0.01, 3), 7 * 4 * NP),
    ]
    rows = []
    for name, call, nbytes in cases:
        for _ in range(3):
            call()
        ts = []
        for _ in range(9):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            call()
            b.record(stream)
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        us = float(np.median(ts))
        gbs = nbytes / us / 1e3
        rows.append({"kernel": name, "us": us, "bytes": nbytes, "gbs": gbs, "frac_hbm": gbs / peaks["hbm_gbs"]})
        print(f"{name:32s} {us:7.1f} us  {nbytes / 1e6:7.1f} MB  {gbs:7.1f} GB/s ({100 * gbs / peaks['hbm_gbs']:5.1f} % of {peaks['hbm_gbs']:.0f})",
              file=sys.stderr, flush=True)
    eng.close()
    print(json.dumps({"glue": rows, "peaks": peaks, "timing": "CUDA events around one call, median of 9 after 3 warm-up calls, 256 MiB "
                      "written between calls"}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA graph replays")
    ap.add_argument("--e2e-sync", action="store_true", help="end-to-end leg with synchronous host-buffer calls")
    ap.add_argument("--zero-dx", action="store_true", help="zero-fill dX before each backward and accumulate into it")
    ap.add_argument("--overlap", action="store_true", help="one all-reduce per projection group beside the rest of the backward "
                    "(gt_dp_allreduce_begin/_end) instead of one after it; measured slower on a single layer (four small "
                    "collectives, and their CTAs cannot share an SM with a GEMM CTA)")
    ap.add_argument("--q4km", action="store_true", help="v and down in Q6_K (the Q4_K_M mix of the second workload) instead of all Q4_K")
    ap.add_argument("--no-group", action="store_true", help="one call per projection instead of q,k,v and gate,up groups")
    ap.add_argument("--sweep", action="store_true", help="token-count sweep of the Q4_K_M projection set instead of the step benchmark")
    ap.add_argument("--glue", action="store_true", help="HBM throughput of the layer-glue kernels instead of the step benchmark")
    ap.add_argument("--sweep-m", type=int, nargs="+", default=[1, 16, 128, 512, 2048])
    ap.add_argument("--e2e-steps", type=int, default=50, help="timed steps of the end-to-end (host-buffer) leg, after 5 warm steps")
    ap.add_argument("--sustained-steps", type=int, default=800, help="steps of the second, long measurement that the clock samples cover")
    ap.add_argument("--no-train-step", action="store_true", help="skip the 28-layer training-step leg (tokens/s)")
    ap.add_argument("--train-steps", type=int, default=10, help="timed steps of the training-step leg")
    ap.add_argument("--train-layers", type=int, default=28, help="layers of the training-step model (28 = the workload)")
    ap.add_argument("--workload", choices=["layer", "step"], default="layer",
                    help="layer: the seven projections of one layer (the headline metric); step: the 28-layer training step (tokens/s)")
    ap.add_argument("--launch-list", action="store_true", help="eager warm-up + steps only (for a profiler's launch list); prints no benchmark value")
    ap.add_argument("--no-parity", action="store_true", help="skip the comparison of the last step's outputs with the CPU path")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
        return
    if args.glue:
        run_glue(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
