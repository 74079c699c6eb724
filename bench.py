#!/usr/bin/env python
"""Benchmark of the L1-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  A step is one forward + one backward of the operator on one batch of
synthetic, seeded inputs (no dataset exists for this path; the shapes ARE the workload):

  dense_cfg2   q,k ~ N(0,1) fp32 [16,1024,16,64], d_attn ~ N(0,1) [16,1024,1024,16]   (default; the
               configuration the headline metric is quoted on)
  dense_cfg3   [2,4096,8,128]
  sparse_cfg4  bs 8, 4096 tokens, 8 heads, width 64, 131072 edges (self edge + 31 random srcs per dst)

metric: dense  Gop/s          = B*H*T^2*W / (t_fwd + t_bwd), one op = one |q-k| term
        sparse Gedge-inst/s   = cl*bs*H   / (t_fwd + t_bwd)

value  : device-resident inputs, CUDA-event timed, max over ranks.
e2e    : the same step through the C ABI's host-buffer entry points (pinned host memory in,
         host memory out; copies inside the timed region; batch items pipelined over the
         library's streams).
N > 1  : one process per GPU (torchrun); every rank runs the full workload on its own data
         (weak scaling; the path has no cross-shard reduction, so no data-path collective);
         value = units of all ranks / slowest rank's time.  "strong" in the same line: the
         workload's ONE batch split over the ranks ((batch, head group) for dense; batch items,
         or dst-token ranges with one all_reduce of d_k, d_v when there are fewer items than
         ranks, for sparse).
Extra keys of the default run (--no-extras drops them): "sparse_cfg4" (the sparse workload's
own record), "reference_cuda" (the reference's GPU extension rebuilt for sm_100, same tensors,
when it was built into oracle/_ref), "module_ms" (the step through the torch.autograd modules).
--impl reference : the reference's own CPU implementation (compiled from its sources into
         oracle/_ref, else the C restatement) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "l1-attention_b200"))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "dense_cfg2": dict(kind="dense", shape=(16, 1024, 16, 64)),
    "dense_cfg3": dict(kind="dense", shape=(2, 4096, 8, 128)),
    "dense_cfg1": dict(kind="dense", shape=(4, 128, 8, 64)),
    "dense_long1": dict(kind="dense", shape=(1, 4096, 8, 128)),  # one long-context item: on 4 GPUs the ranks tile its scores 2 x 2
    "dense_small": dict(kind="dense", shape=(2, 1024, 16, 64)),  # profiling size: 134 MB of scores, > L2
    "sparse_small": dict(kind="sparse", shape=(2, 4096, 8, 64), fan=31),
    "sparse_cfg4": dict(kind="sparse", shape=(8, 4096, 8, 64), fan=31),
    # the dense scores fused with softmax and the value product (no [B,T,T,H] tensor): benchmark and long-context shapes
    "fused_cfg2": dict(kind="fused", shape=(16, 1024, 16, 64)),
    "fused_cfg3": dict(kind="fused", shape=(2, 4096, 8, 128)),
    "fused_small": dict(kind="fused", shape=(2, 1024, 16, 64)),
    # training step of a 4-layer pre-LN transformer on L1AttnSparseBidi (d_model 256, 8 heads x 32, sequence 256,
    # batch 64, vocabulary 64, 16 random srcs per dst + self edge, AdamW); the reference ships no such model
    "train_cfg5": dict(kind="train", batch=64, seq=256, d_model=256, heads=8, layers=4, vocab=64, fan=16),
}
SM_COUNT, FP32_LANES = 148, 128


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], sm_max_mhz=d.get("sm_max_mhz", 1965.0), source="measured")
    return dict(hbm_gbs=6650.0, sm_max_mhz=1965.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def window(self, t0, t1):
        rows = [r for t, r in self.rows if t0 <= t <= t1] or [r for _, r in self.rows[-3:]]
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": len(rows)}
        try:
            sm = sorted(float(r[0]) for r in rows)
            out["sm_mhz"] = sm[len(sm) // 2]
            out["sm_max_mhz"] = float(rows[0][1])
            out["power_w_max"] = max(float(r[2]) for r in rows)
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            out["reasons"] = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        except (IndexError, ValueError):
            pass
        return out

    def stop(self):
        if self.proc:
            self.proc.terminate()


def bench_graph(n, fan, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    r = torch.rand(n, n, generator=g)
    r.fill_diagonal_(2)
    src = r.argsort(1)[:, :fan]
    rows = torch.cat([torch.stack([torch.arange(n).repeat_interleave(fan), src.reshape(-1)], 1),
                      torch.stack([torch.arange(n), torch.arange(n)], 1)])
    return rows[torch.randperm(rows.shape[0], generator=g)]


# ----------------------------------------------------------------------------- reference / CPU arm

def cpu_reference_rate(kind, shape, budget_s, fan=31):
    """Time the reference's CPU implementation on a bounded sample; returns (rate in G units/s, info)."""
    import numpy as np
    import torch
    refdir = os.path.join(ROOT, "oracle", "_ref")
    have_ref = os.path.exists(os.path.join(refdir, "l1attn_drv_cpp.so"))
    if have_ref:
        sys.path.insert(0, refdir)
        import l1attn_drv_cpp
        import l1attn_sparse_drv
        kind_name, dt = "reference", "f64 (the reference CPU extension is float64-only; same seeded values cast up)"
    else:
        from oracle import oracle
        kind_name, dt = "port", "f64"
    bs, n, h, w = shape
    gen = torch.Generator().manual_seed(2000)

    def run_dense(t):
        q = torch.randn(1, t, h, w, generator=gen, dtype=torch.float32).double()
        k = torch.randn(1, t, h, w, generator=gen, dtype=torch.float32).double()
        g = torch.randn(1, t, t, h, generator=gen, dtype=torch.float32).double()
        t0 = time.perf_counter()
        if have_ref:
            l1attn_drv_cpp.forward(q, k)
            l1attn_drv_cpp.backward(g, q, k)
        else:
            oracle.dense_fwd(q.numpy(), k.numpy())
            oracle.dense_bwd(g.numpy(), q.numpy(), k.numpy())
        return time.perf_counter() - t0, float(h) * t * t * w

    def run_sparse(b):
        co = bench_graph(n, fan, 4001)
        from oracle import oracle as orc
        coo_np, dm, _ = orc.expand_coo(co.numpy())
        coo = torch.from_numpy(coo_np)
        q, k, v, dvo = (torch.randn(b, n, h, w, generator=gen, dtype=torch.float32).double() for _ in range(4))
        t0 = time.perf_counter()
        if have_ref:
            vo, attn = l1attn_sparse_drv.forward(v, q, k, coo, dm, True)
            l1attn_sparse_drv.backward(dvo, v, q, k, coo, attn, dm, True)
        else:
            vo, attn = orc.sparse_fwd(v.numpy(), q.numpy(), k.numpy(), coo_np, dm, True)
            orc.sparse_bwd(dvo.numpy(), v.numpy(), q.numpy(), k.numpy(), coo_np, attn, dm, True)
        return time.perf_counter() - t0, float(coo.shape[0]) * b * h

    if kind == "dense":
        run_dense(64)  # warm-up (first call pays page faults / lazy init)
        t_probe, u_probe = run_dense(128)
        t = 128
        while t * 2 <= n and t_probe * ((t * 2) / 128.0) ** 2 <= budget_s:
            t *= 2
        el, units = (t_probe, u_probe) if t == 128 else run_dense(t)
        sample = "one batch item, first %d of %d tokens (B=1,T=%d,H=%d,W=%d), fwd+bwd, %s" % (t, n, t, h, w, dt)
    else:
        el, units = run_sparse(1)
        sample = "one of %d batch items at full graph size (n_tok=%d, %d edges), fwd+bwd, %s" % (bs, n, n * (fan + 1), dt)
    return units / el / 1e9, dict(kind=kind_name, cores=1, sample=sample, seconds=round(el, 3))


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, shape = wl["kind"], wl["shape"]
    per_step = max(1.0, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    rates, info = [], None
    for i in range(args.warmup + args.steps):
        r, info = cpu_reference_rate(kind, shape, per_step, wl.get("fan", 31))
        if i >= args.warmup:
            rates.append(r)
    val = sum(rates) / len(rates)
    unit = "Gop/s" if kind == "dense" else "Gedge-inst/s"
    bs, n, h, w = shape
    units_full = float(bs) * h * n * n * w if kind == "dense" else float(n * (wl.get("fan", 31) + 1)) * bs * h
    line = {
        "impl": "reference", "metric": metric_name(kind), "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": units_full / (val * 1e9) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": config_of(args, wl),
        "cpu_baseline": dict(value=val, unit=unit, cores=info["cores"], kind=info["kind"], sample=info["sample"]),
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "ms_per_step is the full workload extrapolated from the sampled rate",
    }
    print(json.dumps(line), flush=True)


def metric_name(kind):
    return "dense L1Attn fwd+bwd Gop/s (B*H*T^2*W)" if kind == "dense" else "sparse COO L1AttnSparse fwd+bwd edge-instances/s"


def config_of(args, wl):
    bs, n, h, w = wl["shape"]
    strong = getattr(args, "scaling", "weak") == "strong"
    c = {"workload": "%s: %s" % (args.workload, "x".join(map(str, wl["shape"]))),
         "per_gpu_batch": bs / args.gpus if strong else bs,
         "global_batch": bs if strong else bs * args.gpus, "n_tok": n, "heads": h, "width": w,
         "partition": "independent batch items per GPU, no collective",
         "l2": "per-step working set (>= 2 GiB dense, 0.8 GB sparse) exceeds the 126 MB L2; no flush"}
    if wl["kind"] == "sparse":
        c["edges"] = n * (wl["fan"] + 1)
    return c


def time_reference_cuda(kind, dev, v):
    """CUDA-event time of the reference's GPU extension (its operator cost: transposes, memsets, atomics)."""
    import importlib
    import torch
    refdir = os.path.join(ROOT, "oracle", "_ref")
    name = "ref_l1attn_cuda_drv" if kind == "dense" else "ref_l1attn_sparse_cuda_drv"
    if not os.path.exists(os.path.join(refdir, name + ".so")):
        return {"unavailable": "oracle/_ref/%s.so not built" % name}
    sys.path.insert(0, refdir)
    drv = importlib.import_module(name)
    if kind == "dense":
        fwd = lambda: drv.forward(v["q"], v["k"])
        bwd = lambda: drv.backward(v["g"], v["q"], v["k"])
    else:
        attn_ref = drv.forward(v["v"], v["q"], v["k"], v["coo"], v["dm"], True)[1]
        fwd = lambda: drv.forward(v["v"], v["q"], v["k"], v["coo"], v["dm"], True)
        bwd = lambda: drv.backward(v["dvo"], v["v"], v["q"], v["k"], v["coo"], attn_ref, v["dm"], True)
    out = {}
    for nm, f in (("fwd_ms", fwd), ("bwd_ms", bwd)):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            f()
        e1.record()
        torch.cuda.synchronize()
        out[nm] = e0.elapsed_time(e1) / 5
    out["speedup"] = (out["fwd_ms"] + out["bwd_ms"]) / (v["fwd_ms"] + v["bwd_ms"])
    out["note"] = "reference cuda/ extension rebuilt for sm_100 with its own flags, same tensors, CUDA events"
    return out


# ----------------------------------------------------------------------------- config-5 training step

def build_transformer(wl, attn_fn, dev):
    """4-layer pre-LayerNorm transformer; attention = L1AttnSparseBidi over a fixed random graph.
    attn_fn(vf, vb, q, k) -> vo, all [batch, seq, heads, width]."""
    import torch
    from torch import nn
    d, hds, width = wl["d_model"], wl["heads"], wl["d_model"] // wl["heads"]

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.qkv = nn.Linear(d, 4 * d)  # q, k, vf, vb
            self.wo = nn.Linear(d, d)
            self.mlp = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d))

        def forward(self, x):
            b, t, _ = x.shape
            q, k, vf, vb = (y.reshape(b, t, hds, width) for y in self.qkv(self.ln1(x)).chunk(4, -1))
            x = x + self.wo(attn_fn(vf, vb, q, k).reshape(b, t, d))
            return x + self.mlp(self.ln2(x))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok, self.pos = nn.Embedding(wl["vocab"], d), nn.Parameter(torch.zeros(wl["seq"], d))
            self.blocks = nn.ModuleList(Block() for _ in range(wl["layers"]))
            self.ln, self.head = nn.LayerNorm(d), nn.Linear(d, wl["vocab"])

        def forward(self, idx):
            x = self.tok(idx) + self.pos
            for blk in self.blocks:
                x = blk(x)
            return self.head(self.ln(x))

    torch.manual_seed(5005)
    return Model().to(dev)


def run_train(args, wl):
    import torch
    import torch.nn.functional as F
    import l1attn_sparse_cuda
    import l1attn_sparse_bidi_cuda

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device -- this library has no CPU path")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    n = wl["seq"]
    co = bench_graph(n, wl["fan"], 5001)
    graph = l1attn_sparse_cuda.SparseGraph(co, device=dev)
    g = torch.Generator().manual_seed(5002)
    tokens = torch.randint(0, wl["vocab"], (wl["batch"], n), generator=g).to(dev)
    targets = torch.randint(0, wl["vocab"], (wl["batch"], n), generator=g).to(dev)

    def timed(attn_fn, steps, warmup):
        model = build_transformer(wl, attn_fn, dev)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
        losses = []

        def step():
            opt.zero_grad(set_to_none=True)
            loss = F.cross_entropy(model(tokens).reshape(-1, wl["vocab"]), targets.reshape(-1))
            loss.backward()
            opt.step()
            return loss

        for _ in range(max(warmup, 3)):
            losses.append(float(step().detach()))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            loss = step()
        e1.record()
        torch.cuda.synchronize()
        losses.append(float(loss.detach()))
        return e0.elapsed_time(e1) / steps, losses

    def timed_graph(attn_fn, steps, warmup):
        """The same step captured once into a CUDA graph and replayed (whole-network capture: forward,
        backward and the AdamW update; static input tensors).  Works because the operators launch on the
        current stream, take their edge index from the prebuilt graph object and never synchronise."""
        model = build_transformer(wl, attn_fn, dev)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, capturable=True)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                opt.zero_grad(set_to_none=True)
                F.cross_entropy(model(tokens).reshape(-1, wl["vocab"]), targets.reshape(-1)).backward()
                opt.step()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        opt.zero_grad(set_to_none=True)
        with torch.cuda.graph(g):
            loss = F.cross_entropy(model(tokens).reshape(-1, wl["vocab"]), targets.reshape(-1))
            loss.backward()
            opt.step()
        losses = []
        for _ in range(max(warmup, 3)):
            g.replay()
            losses.append(float(loss.detach()))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        losses.append(float(loss.detach()))
        return e0.elapsed_time(e1) / steps, losses

    ours = lambda vf, vb, q, k: graph.attend_bidi(vf, vb, q, k)
    ms, losses = timed(ours, args.steps, args.warmup)
    line = {"metric": "training tokens/s, 4-layer pre-LN transformer with L1AttnSparseBidi (config 5)",
            "value": wl["batch"] * n / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "train_cfg5", **{k: v for k, v in wl.items() if k != "kind"},
                       "edges": int(graph.n_edges), "dst_mxlen": int(graph.dst_mxlen), "optimizer": "AdamW"},
            "loss_first": losses[0], "loss_last": losses[-1]}
    if args.cuda_graph:
        gms, gl = timed_graph(ours, args.steps, args.warmup)
        line["cuda_graph"] = {"ms_per_step": gms, "tokens_per_s": wl["batch"] * n / (gms * 1e-3), "loss_last": gl[-1],
                              "note": "one captured graph per step (forward, backward, AdamW), replayed"}
    if args.compare_reference_cuda:
        refdir = os.path.join(ROOT, "oracle", "_ref")
        if os.path.exists(os.path.join(refdir, "ref_l1attn_sparse_bidi_cuda_drv.so")):
            sys.path.insert(0, refdir)
            import ref_l1attn_sparse_bidi_cuda_drv as refdrv

            class RefFn(torch.autograd.Function):  # the reference's autograd glue (cuda/l1attn_sparse_bidi_cuda.py:8-48)
                @staticmethod
                def forward(ctx, vf, vb, q, k):
                    vf, vb, q, k = (t.contiguous() for t in (vf, vb, q, k))
                    vo, attn = refdrv.forward(vf, vb, q, k, graph.coo, graph.dst_mxlen, True)
                    ctx.save_for_backward(vf, vb, q, k, attn)
                    return vo

                @staticmethod
                def backward(ctx, dvo):
                    vf, vb, q, k, attn = ctx.saved_tensors
                    return tuple(refdrv.backward(dvo.contiguous(), vf, vb, q, k, graph.coo, attn, graph.dst_mxlen, True))

            rms, rl = timed(lambda vf, vb, q, k: RefFn.apply(vf, vb, q, k), args.steps, args.warmup)
            line["reference_cuda"] = {"ms_per_step": rms, "tokens_per_s": wl["batch"] * n / (rms * 1e-3),
                                      "speedup": rms / ms, "loss_last": rl[-1]}
    print(json.dumps(line), flush=True)


def run_fused(args, wl):
    """Forward and forward+backward of l1attn_fused_cuda.L1AttnSoftmaxV beside the unfused chain the
    reference's callers write (library scores -> torch softmax -> torch einsum), with peak memory."""
    import torch
    import l1attn_cabi
    import l1attn_cuda
    import l1attn_fused_cuda

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device -- this library has no CPU path")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    bs, n, h, w = wl["shape"]
    gen = torch.Generator(device=dev).manual_seed(6001)
    q, k = (0.3 * torch.randn(bs, n, h, w, device=dev, generator=gen) for _ in range(2))
    v, g = (torch.randn(bs, n, h, w, device=dev, generator=gen) for _ in range(2))
    warm = max(args.warmup, 3)

    def timed(fn):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats(dev)
        base = torch.cuda.memory_allocated(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps, (torch.cuda.max_memory_allocated(dev) - base) / 2 ** 20

    out = torch.empty_like(v)
    fwd_ms, _ = timed(lambda: l1attn_cabi.dense_softmax_v_fwd(q, k, v, "softmax", out=out))
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    fused_mod = l1attn_fused_cuda.L1AttnSoftmaxV("softmax")
    dense_mod = l1attn_cuda.L1Attn()

    def fused_step():
        for t in (qr, kr, vr):
            t.grad = None
        fused_mod(qr, kr, vr).backward(g)

    def unfused_step():
        for t in (qr, kr, vr):
            t.grad = None
        torch.einsum("bsdh,bshw->bdhw", torch.softmax(dense_mod(qr, kr), 1), vr).backward(g)

    def unfused_fwd():
        with torch.no_grad():
            torch.einsum("bsdh,bshw->bdhw", torch.softmax(dense_mod(q, k), 1), v)

    step_ms, step_mib = timed(fused_step)
    ufwd_ms, ufwd_mib = timed(unfused_fwd)
    ustep_ms, ustep_mib = timed(unfused_step)
    ops = bs * h * n * n * w
    # forward instruction floor per (t, s, w) term: 1.5 issue slots for the score + 1 FMA of the value
    # product (v_width = width) against 4 issue slots per clock per SM
    sm_mhz, sms = 1965.0, 148
    floor_ms = ops * 2.5 / 32 / (4 * sms * sm_mhz * 1e6) * 1e3
    line = {"metric": "fused dense L1 attention (scores+softmax+V) forward Gop/s (B*H*T^2*W)", "value": ops / (fwd_ms * 1e-3) / 1e9,
            "unit": "Gop/s", "n_gpus": 1, "steps": args.steps, "warmup": warm, "ms_per_step": fwd_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s: %dx%dx%dx%d, v_width %d" % (args.workload, bs, n, h, w, w)},
            "fwd_ms": fwd_ms, "fwd_bwd_ms": step_ms, "fwd_bwd_peak_extra_mib": step_mib,
            "issue_floor": {"ms": floor_ms, "frac": floor_ms / fwd_ms,
                            "model": "2.5 warp instructions per 32 terms, 4 issue slots/clk/SM, 148 SMs, 1965 MHz"},
            "unfused": {"fwd_ms": ufwd_ms, "fwd_peak_extra_mib": ufwd_mib, "fwd_bwd_ms": ustep_ms,
                        "fwd_bwd_peak_extra_mib": ustep_mib,
                        "chain": "l1attn_cuda.L1Attn -> torch.softmax(dim=1) -> torch.einsum('bsdh,bshw->bdhw')"},
            "gpu_launches": args.steps}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm

def _events(torch, n):
    return [torch.cuda.Event(enable_timing=True) for _ in range(n)]


def setup_dense(torch, cabi, shape, dev, seed):
    """Device-resident tensors and the two timed calls of a dense step (outputs and scratch pre-allocated)."""
    bs, n, h, w = shape
    gen = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(shape, generator=gen, device=dev)
    k = torch.randn(shape, generator=gen, device=dev)
    g = torch.randn((bs, n, n, h), generator=gen, device=dev)
    attn = torch.empty((bs, n, n, h), device=dev)
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    scratch = torch.empty(cabi.lib().l1attn_dense_bwd_scratch_bytes(bs, n, h, w, 0), dtype=torch.uint8, device=dev)
    return dict(kind="dense", shape=shape, q=q, k=k, g=g, units=float(bs) * h * n * n * w,
                launches=DENSE_LAUNCHES_PER_STEP,
                fwd=lambda: cabi.dense_fwd(q, k, out=attn),
                bwd=lambda: cabi.dense_bwd(g, q, k, out=(dq, dk), scratch=scratch))


def setup_sparse(torch, cabi, shape, fan, dev, seed, qk_scale):
    bs, n, h, w = shape
    gen = torch.Generator(device=dev).manual_seed(seed)
    co = bench_graph(n, fan, 4001)
    coo_h, dm, _ = cabi.expand_coo_host(co.numpy())
    coo = torch.from_numpy(coo_h).to(dev)
    index = cabi.SparseIndex(coo, n, dm)
    index.check()
    q, k = (qk_scale * torch.randn(shape, generator=gen, device=dev) for _ in range(2))
    v, dvo = (torch.randn(shape, generator=gen, device=dev) for _ in range(2))
    vo = torch.empty_like(v)
    attn = torch.empty((bs, n, dm, h), device=dev)
    grads = (torch.empty_like(v), None, torch.empty_like(q), torch.empty_like(k))
    scratch = torch.empty_like(attn)
    return dict(kind="sparse", shape=shape, q=q, k=k, v=v, dvo=dvo, coo=coo, coo_h=coo_h, dm=dm, attn=attn, fan=fan,
                units=float(coo.shape[0]) * bs * h, launches=4, qk_scale=qk_scale,
                fwd=lambda: cabi.sparse_fwd(v, q, k, index, True, out=(vo, attn)),
                bwd=lambda: cabi.sparse_bwd(dvo, v, q, k, index, attn, True, out=grads, scratch=scratch))


def time_steps(torch, wl, steps, warmup, sync_all):
    """CUDA events on the launching stream around every forward and backward of `steps` steps."""
    for _ in range(max(warmup, 3)):
        wl["fwd"]()
        wl["bwd"]()
    sync_all()
    ev = [_events(torch, 3) for _ in range(steps)]
    for i in range(steps):
        ev[i][0].record()
        wl["fwd"]()
        ev[i][1].record()
        wl["bwd"]()
        ev[i][2].record()
    sync_all()
    return dict(total_ms=ev[0][0].elapsed_time(ev[-1][2]),
                fwd_ms=sum(e[0].elapsed_time(e[1]) for e in ev) / steps,
                bwd_ms=sum(e[1].elapsed_time(e[2]) for e in ev) / steps)


def e2e_setup(torch, cabi, wl):
    """The same step through the host-buffer C ABI from pinned host memory; returns (step(), h2d, d2h bytes)."""
    shape = wl["shape"]
    bs, n, h, w = shape
    if wl["kind"] == "dense":
        hq, hk = (torch.randn(shape).pin_memory() for _ in range(2))
        hg = torch.randn((bs, n, n, h)).pin_memory()
        hattn = torch.empty((bs, n, n, h)).pin_memory()
        hdq, hdk = torch.empty(shape).pin_memory(), torch.empty(shape).pin_memory()
        nqk, na = hq.numel() * 4, hg.numel() * 4

        def step():
            # the upstream gradient of this workload does not depend on the scores, so the two calls are
            # enqueued together: the backward's copies in overlap the forward's copy out (full-duplex PCIe)
            cabi.dense_fwd_host(hq.numpy(), hk.numpy(), out=hattn.numpy(), wait=False)
            cabi.dense_bwd_host(hg.numpy(), hq.numpy(), hk.numpy(), out=(hdq.numpy(), hdk.numpy()), wait=False)
            cabi.host_sync()
            return float(hdq[0, 0, 0, 0])
        return step, 2 * nqk + (na + 2 * nqk), na + 2 * nqk
    hq, hk, hv, hdvo = (torch.randn(shape).pin_memory() for _ in range(4))
    hq.mul_(wl["qk_scale"])
    hk.mul_(wl["qk_scale"])
    hvo, hdv, hdq, hdk = (torch.empty(shape).pin_memory() for _ in range(4))
    hattn = torch.empty(tuple(wl["attn"].shape)).pin_memory()
    coo_np, dm = wl["coo_h"], wl["dm"]
    nqk, na, nc = hq.numel() * 4, hattn.numel() * 4, coo_np.nbytes

    def step():
        _, attn_h = cabi.sparse_fwd_host(hv.numpy(), hq.numpy(), hk.numpy(), coo_np, dm, True, out=(hvo.numpy(), hattn.numpy()))
        r = cabi.sparse_bwd_host(hdvo.numpy(), hv.numpy(), hq.numpy(), hk.numpy(), coo_np, attn_h, dm, True,
                                 out=(hdv.numpy(), None, hdq.numpy(), hdk.numpy()))
        return float(r[0][0, 0, 0, 0])
    return step, (3 * nqk + nc) + (4 * nqk + na + nc), (nqk + na) + 3 * nqk


def time_e2e(torch, step, n_steps):
    step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_steps):
        step()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) * 1e3 / n_steps


def l2_copy_rate(torch, dev):
    """GB/s (read + write) of a device copy whose 2 x 24 MiB working set stays in the 126 MB L2: the yardstick
    for the sparse kernels' row gathers, which hit L2 (every operand of the sparse config is 67 MB)."""
    a = torch.empty(6 << 20, device=dev)
    b = torch.empty_like(a)
    for _ in range(5):
        b.copy_(a)
    e0, e1 = _events(torch, 2)
    e0.record()
    for _ in range(20):
        b.copy_(a)
    e1.record()
    torch.cuda.synchronize()
    return 20 * 2 * a.numel() * 4 / (e0.elapsed_time(e1) * 1e-3) / 1e9


def roofline_of(wl, t, pk, clocks, l2_gbs=None):
    """(roofline, alu_roofline) of a timed workload; t = dict(fwd_ms, bwd_ms)."""
    bs, n, h, w = wl["shape"]
    fwd_ms, bwd_ms = t["fwd_ms"], t["bwd_ms"]
    if wl["kind"] == "dense":
        # dominant kernel: the single-visit backward (dense_bwd_sv_kernel; the CUDA-event time bwd_ms also holds the tie
        # detector, the sum of the d_k shares and the tie fix, ~8 % of it).  Algorithmic HBM bytes per backward: d_attn,
        # q and k read once, both gradients written once.
        alg_bytes = 4.0 * (bs * n * n * h + 4 * bs * n * h * w)
        roof = {"bound": "hbm", "kernel": "dense_bwd_sv_kernel", "achieved": alg_bytes / (bwd_ms * 1e-3) / 1e9,
                "peak": pk["hbm_gbs"], "unit": "GB/s", "peak_source": pk["source"],
                # ncu dram__bytes_read+write of this kernel at B=2,T=1024,H=16,W=64 (profiles/), scaled by batch
                "traffic": (DENSE_BWD_TRAFFIC_B2 * bs / 2.0) if (n, h, w) == (1024, 16, 64) and DENSE_BWD_TRAFFIC_B2 else None,
                "note": "the kernel is bound by instruction issue, not by HBM: see alu_roofline"}
        roof["frac"] = roof["achieved"] / roof["peak"]
        mhz = (clocks or {}).get("sm_max_mhz") or pk["sm_max_mhz"]
        alu_peak = SM_COUNT * FP32_LANES * mhz * 1e6
        ops = wl["units"]
        alu = {"model": "lane-instructions per op: fwd 2 (sub, abs-add), bwd 3 (sub, two adds)",
               "peak_lane_instr_per_s": alu_peak, "peak_basis": "148 SM x 128 FP32 lanes x %.0f MHz" % mhz,
               "fwd_frac": 2 * ops / (fwd_ms * 1e-3) / alu_peak, "bwd_frac": 3 * ops / (bwd_ms * 1e-3) / alu_peak,
               "fwd_bwd_frac": 5 * ops / ((fwd_ms + bwd_ms) * 1e-3) / alu_peak}
        return roof, alu
    nqk, na, nc = bs * n * h * w * 4.0, wl["attn"].numel() * 4.0, wl["coo"].numel() * 4.0
    alg_bytes = (3 * nqk + nqk + na + nc) + (4 * nqk + na + 3 * nqk + nc)
    roof = {"bound": "hbm", "kernel": "sparse fwd+bwd (4 kernels)", "achieved": alg_bytes / ((fwd_ms + bwd_ms) * 1e-3) / 1e9,
            "peak": pk["hbm_gbs"], "unit": "GB/s", "peak_source": pk["source"],
            # ncu dram__bytes_read+write of the kernels of a step at bs=2 (profiles/sparse_kernels.md), scaled by
            # batch: every batch item streams its own tensors
            "traffic": (SPARSE_TRAFFIC_B2 * bs / 2.0) if (n, h, w, wl["fan"]) == (4096, 8, 64, 31) else None,
            "note": "compulsory bytes (every tensor touched once) summed over the step's kernels; the row gathers hit L2: see gathered"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    # rows fetched per edge instance (cl * bs * H of them): forward k and v of the src; backward v, k of the src in
    # the dst pass and dvo, q of the dst in the src pass -- each a width (or v_width) slice of one head
    gathered = wl["units"] * w * 4.0 * (2 + 4)
    roof["gathered"] = {"bytes_per_step": gathered, "achieved": gathered / ((fwd_ms + bwd_ms) * 1e-3) / 1e9, "unit": "GB/s",
                        "l2_copy_gbs": l2_gbs, "frac_of_l2_copy": (gathered / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / l2_gbs) if l2_gbs else None,
                        "note": "l2_copy_gbs = read+write rate of a torch copy whose working set (48 MiB) stays in L2, measured in this run"}
    return roof, None


# kernels of this library per dense step: forward; tie detector; single-visit backward; sum of the d_k shares;
# two-pass kernel (returns at once unless the tie list overflowed); tie fix
DENSE_LAUNCHES_PER_STEP = 6
# ncu dram__bytes_read.sum + dram__bytes_write.sum per launch at the profiling sizes (profiles/*.md)
DENSE_BWD_TRAFFIC_B2 = 198.8e6
SPARSE_TRAFFIC_B2 = 226.9e6


def module_step_ms(torch, wl, steps):
    """The same step through the drop-in autograd modules a user of the reference calls (l1attn_cuda.L1Attn /
    l1attn_sparse_cuda.L1AttnSparse + .backward): output, gradient and scratch allocations included."""
    if wl["kind"] == "dense":
        import l1attn_cuda
        mod = l1attn_cuda.L1Attn()
        q, k = (wl[x].clone().requires_grad_(True) for x in ("q", "k"))

        def step():
            q.grad = k.grad = None
            mod(q, k).backward(wl["g"])
    else:
        import l1attn_sparse_cuda
        mod = l1attn_sparse_cuda.L1AttnSparse()
        v, q, k = (wl[x].clone().requires_grad_(True) for x in ("v", "q", "k"))

        def step():
            v.grad = q.grad = k.grad = None
            mod(v, q, k, wl["coo"], wl["dm"], True).backward(wl["dvo"])
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = _events(torch, 2)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_ours(args, wl):
    import torch
    import torch.distributed as dist
    import l1attn_cabi as cabi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device -- this library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cabi.lib()
    import l1attn_shard as shard
    kind, shape = wl["kind"], wl["shape"]
    if args.scaling == "strong":  # the workload's batch items are dealt out to the ranks
        lo, hi = shard.shard_range(shape[0], rank, world)
        if hi == lo:
            raise SystemExit("bench.py: more ranks than batch items in --scaling strong")
        shape = (hi - lo,) + tuple(shape[1:])
    pk = peaks()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def all_units(units):  # units of every rank (ranks may hold different batch counts under strong scaling)
        if world == 1:
            return units
        tu = torch.tensor([units], device=dev, dtype=torch.float64)
        dist.all_reduce(tu)
        return float(tu.item())

    def make(kind_, shape_, fan=31):
        if kind_ == "dense":
            return setup_dense(torch, cabi, shape_, dev, 2000 + rank)
        return setup_sparse(torch, cabi, shape_, fan, dev, 4100 + rank, args.qk_scale)

    def measure(w_, steps, e2e_steps):
        """Device-resident timing (max over ranks) and the end-to-end leg of one workload -> record."""
        t = time_steps(torch, w_, steps, args.warmup, sync_all)
        ms = shard.max_over_ranks(t["total_ms"], dev) / steps
        units = all_units(w_["units"])
        rec = dict(value=units / (ms * 1e-3) / 1e9, ms_per_step=ms, fwd_ms=t["fwd_ms"], bwd_ms=t["bwd_ms"], t=t)
        if not args.kernel_only:
            step, h2d, d2h = e2e_setup(torch, cabi, w_)
            sync_all()
            ems = shard.max_over_ranks(time_e2e(torch, step, e2e_steps), dev)
            rec["e2e"] = {"value": units / (ems * 1e-3) / 1e9, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                          "ms_per_step": ems, "steps": e2e_steps,
                          "h2d_plus_d2h_gbs_per_rank": (h2d + d2h) / (ems * 1e-3) / 1e9}
            cabi.lib().l1attn_host_release()
        return rec

    sampler = ClockSampler(local) if rank == 0 else None
    t_wall0 = time.time()
    main_wl = make(kind, shape, wl.get("fan", 31))
    e2e_steps = max(1, min(args.steps, 3))
    rec = measure(main_wl, args.steps, e2e_steps)
    clocks = sampler.window(t_wall0, time.time()) if sampler else None
    unit = "Gop/s" if kind == "dense" else "Gedge-inst/s"
    secondary = not args.kernel_only and not args.no_extras
    line = None
    if rank == 0:
        roof, alu = roofline_of(main_wl, rec["t"], pk, clocks, None if kind == "dense" else l2_copy_rate(torch, dev))
        cpu = None
        if world == 1 and not args.no_cpu_baseline and not args.kernel_only:
            r, info = cpu_reference_rate(kind, shape, 15.0, wl.get("fan", 31))
            cpu = dict(value=r, unit=unit, cores=info["cores"], kind=info["kind"], sample=info["sample"])
        e2e = rec.get("e2e") or {"value": 0.0, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "ms_per_step": 0.0, "steps": 0}
        e2e["unit"] = unit
        line = {
            "metric": metric_name(kind), "value": rec["value"], "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_of(args, wl),
            "fwd_ms": rec["fwd_ms"], "bwd_ms": rec["bwd_ms"], "roofline": roof, "alu_roofline": alu, "cpu_baseline": cpu,
            "e2e": e2e, "gpu_launches": main_wl["launches"] * args.steps, "clocks": clocks,
        }
        if secondary:
            line["module_ms"] = module_step_ms(torch, main_wl, min(args.steps, 10))
        if secondary or args.compare_reference_cuda:
            line["reference_cuda"] = time_reference_cuda(kind, dev, dict(main_wl, fwd_ms=rec["fwd_ms"], bwd_ms=rec["bwd_ms"]))
    del main_wl
    torch.cuda.empty_cache()

    # ---- the second half of the metric: the sparse config on every rank (weak), in the same line
    if secondary and kind == "dense":
        swl_cfg = WORKLOADS["sparse_cfg4"]
        swl = make("sparse", swl_cfg["shape"], swl_cfg["fan"])
        srec = measure(swl, args.steps, e2e_steps)
        if rank == 0:
            sroof, _ = roofline_of(swl, srec["t"], pk, clocks, l2_copy_rate(torch, dev))
            srec.pop("t")
            srec.update(metric=metric_name("sparse"), unit="Gedge-inst/s", roofline=sroof, gpu_launches=swl["launches"] * args.steps,
                        config={"workload": "sparse_cfg4: 8x4096x8x64, 131072 edges, dst_mxlen %d" % swl["dm"],
                                "values": "q,k ~ %g N(0,1); v, dvo ~ N(0,1)" % args.qk_scale,
                                "per_gpu_batch": 8, "global_batch": 8 * world})
            srec["e2e"]["unit"] = "Gedge-inst/s"
            if world == 1 and not args.no_cpu_baseline:
                r, info = cpu_reference_rate("sparse", swl_cfg["shape"], 15.0, swl_cfg["fan"])
                srec["cpu_baseline"] = dict(value=r, unit="Gedge-inst/s", cores=info["cores"], kind=info["kind"], sample=info["sample"])
            srec["module_ms"] = module_step_ms(torch, swl, min(args.steps, 10))
            srec["reference_cuda"] = time_reference_cuda("sparse", dev, dict(swl, fwd_ms=srec["fwd_ms"], bwd_ms=srec["bwd_ms"]))
            line["sparse_cfg4"] = srec
        del swl
        torch.cuda.empty_cache()
        if world > 1:
            st = run_strong(torch, dist, cabi, shard, args, swl_cfg, rank, world, dev, sync_all)
            if rank == 0:
                line["sparse_cfg4"]["strong"] = st

    # ---- strong scaling beside the weak number: the SAME global workload dealt out over the ranks
    if not args.no_extras and world > 1 and args.scaling == "weak":
        line_strong = run_strong(torch, dist, cabi, shard, args, wl, rank, world, dev, sync_all)
        if rank == 0:
            line["strong"] = line_strong

    if rank == 0:
        print(json.dumps(line), flush=True)
    if sampler:
        sampler.stop()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_strong(torch, dist, cabi, shard, args, wl, rank, world, dev, sync_all):
    """The workload at its stated global size, partitioned over the ranks (l1attn_shard): dense by (batch, head
    group) with shard-resident outputs and no collective -- with fewer batch items than ranks also by square
    blocks of an item's scores (one all-reduce each of d_q and d_k), reporting the faster; sparse by batch item when there are enough of them,
    else by dst-token range with ONE all-reduce of d_k and d_v.  Returns the record for rank 0."""
    kind, shape = wl["kind"], wl["shape"]
    bs, n, h, w = shape
    unit = "Gop/s" if kind == "dense" else "Gedge-inst/s"
    if kind == "dense":
        units = float(bs) * h * n * n * w
        out = {}
        if bs < world:
            # fewer batch items than ranks: also the square-block partition (all heads of the kernels' work items
            # stay busy; d_q and d_k partial sums meet in one all-reduce each)
            plan = shard.DenseGridShard(bs, n, h, rank, world)
        if bs < world and any(len(p["row"]) > 1 for p in plan.part):  # (else it is the head-group split below; same answer on every rank)
            m = plan.me
            lshape = (m["b1"] - m["b0"], m["t1"] - m["t0"], m["h1"] - m["h0"], w)
            gwl = setup_dense(torch, cabi, lshape, dev, 2000 + rank)
            gattn = torch.empty((lshape[0], lshape[1], lshape[1], lshape[2]), device=dev)
            gout = (torch.empty_like(gwl["q"]), torch.empty_like(gwl["k"]))
            gwl["fwd"] = lambda: plan.forward(gwl["q"], gwl["k"], out=gattn)
            gwl["bwd"] = lambda: plan.backward(gwl["g"], gwl["q"], gwl["k"], out=gout)
            t = time_steps(torch, gwl, args.steps, args.warmup, sync_all)
            ms = shard.max_over_ranks(t["total_ms"], dev) / args.steps
            out["grid"] = {"value": units / (ms * 1e-3) / 1e9, "unit": unit, "ms_per_step": ms,
                           "fwd_ms": shard.max_over_ranks(t["fwd_ms"], dev), "bwd_ms": shard.max_over_ranks(t["bwd_ms"], dev),
                           "partition": "square blocks: " + plan.describe(), "collective": plan.collective_note()}
            del gwl, gattn, gout
        b0, b1, h0, h1 = shard.dense_partition(bs, h, world)[rank]
        swl = setup_dense(torch, cabi, (b1 - b0, n, h1 - h0, w), dev, 2000 + rank)
        t = time_steps(torch, swl, args.steps, args.warmup, sync_all)
        ms = shard.max_over_ranks(t["total_ms"], dev) / args.steps
        out.update({"value": units / (ms * 1e-3) / 1e9, "unit": unit, "ms_per_step": ms, "collective": None,
                    "partition": "(batch, head group): rank 0 holds batch %d..%d, heads %d..%d of %s; outputs stay on their rank"
                                 % (b0, b1, h0, h1, list(shape))})
        if "grid" in out and out["grid"]["value"] > out["value"]:  # report the better partition as the strong-scaling figure
            out = dict(out["grid"], head_groups={k: out[k] for k in ("value", "ms_per_step", "partition")})
        return out
    import l1attn_sparse_cuda
    co = bench_graph(n, wl["fan"], 4001)
    gen = torch.Generator(device=dev).manual_seed(4100)  # same tensors on every rank (replicated inputs)
    q, k = (args.qk_scale * torch.randn(shape, generator=gen, device=dev) for _ in range(2))
    v, dvo = (torch.randn(shape, generator=gen, device=dev) for _ in range(2))
    units = float(co.shape[0]) * bs * h

    def run(mode):
        plan = shard.SparseShard(co, bs, n, rank, world, device=dev, n_heads=h, mode=mode)
        step = lambda: plan.forward_backward(v, q, k, dvo, True)
        for _ in range(max(args.warmup, 3)):
            step()
        sync_all()
        e0, e1 = _events(torch, 2)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        sync_all()
        ms = shard.max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
        return {"value": units / (ms * 1e-3) / 1e9, "unit": unit, "ms_per_step": ms, "partition": plan.describe(),
                "collective": plan.collective_note()}
    out = run("auto")
    if bs < world:  # also the dst-token-range form with its all-reduce, whichever form "auto" chose
        out["dst_range"] = run("dst")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--compare-reference-cuda", action="store_true",
                    help="also time the reference's own GPU kernels (oracle/_ref, rebuilt for sm_100) on the same inputs")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak (default): every rank runs the full workload on its own data; strong: the "
                         "workload's batch is split across the ranks")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="train_cfg5: also time the step captured into one CUDA graph and replayed")
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end and CPU legs (profiling runs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the records added beside the main workload (sparse config, reference GPU kernels, "
                         "module call, strong scaling)")
    ap.add_argument("--qk-scale", type=float, default=1.0,
                    help="sparse workloads: q,k ~ qk_scale * N(0,1) (1: logits near -9, weights ~1e-4; 0.25: weights ~1/32)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if wl["kind"] == "train":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference ships no model for config 5 and its CPU "
                              "extension has no training loop; use --compare-reference-cuda on the default arm"}))
        else:
            run_train(args, wl)
    elif wl["kind"] == "fused":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no fused operator; its CPU "
                              "arm is measured on the dense workloads"}))
        else:
            run_fused(args, wl)
    elif args.impl == "reference":
        run_reference_arm(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
