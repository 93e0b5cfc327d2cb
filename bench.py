#!/usr/bin/env python
"""Benchmark of the CASTLE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-decode]

N > 1 is launched by torchrun (one rank per GPU); ranks own disjoint (batch, head)
rectangles of the workload and never communicate inside the timed path.

Workload (synthetic, seeded): a single CASTLE attention layer in bf16, B=4, N=4096, H=16,
d_head=64, dim=1024; x ~ N(0,1), default-initialised projections, upstream gradient ~ N(0,1).
One step = forward + backward of the attention core.

  value     whole-job TFLOP/s of the core (forward + backward kernels, q/k/v already in HBM),
            counted with the ALGORITHMIC flops 19 * B*H*N^2*d (5 forward + 14 backward incl.
            recompute); the reference's cubic N^3 term is not credited.
  e2e       the same flops over the time of `Castle(x)` forward + backward called with HOST
            tensors: pinned x and upstream grad copied in, out and dx copied back, projections
            included.
  roofline  the backward main kernel alone, timed with CUDA events recorded around it.
  decode    (secondary) cached single-token decode at B=64, H=16, d=128, prefix 8192, 256 steps.
  cfg4      (secondary) the long-context configuration's per-GPU slice: B=1, N=16384, H=32, d=128.
  cfg3      (secondary, 1 GPU) training step of the 8-layer byte LM on batch 16 x 1024 bytes.

`--impl reference` times the reference's own PyTorch CPU path (its staged copy under oracle/_ref;
the oracle port when that is absent) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(batch=4, seq_len=4096, heads=16, dim_head=64, dim=1024)
DECODE_CFG = dict(batch=64, prefix=8192, heads=16, dim_head=128, dim=2048, steps=256)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(tflops=float(d["bf16_tflops"]), hbm=float(d["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, hbm=6650.0, source="fallback")


def captured_traffic(key, units):
    """DRAM bytes per launch from the ncu summary table under profiles/, scaled to `units` of this launch
    (None when no capture of that kernel and size is on file)."""
    f = ROOT / "profiles" / "ncu_dram_traffic.txt"
    if not f.exists():
        return None
    for ln in f.read_text().splitlines():
        w = ln.split()
        if len(w) >= 3 and w[0] == key:
            return int(float(w[1]) / float(w[2]) * units)
    return None


def core_flops(b, h, n, d):
    u = b * h * n * n * d
    return 5 * u, 14 * u


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thr = None

    def _open(self):
        import pynvml as nv
        nv.nvmlInit()
        idx = self.index
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                idx = int(vis.split(",")[self.index])
            except ValueError:
                pass
        self._nv, self._h = nv, nv.nvmlDeviceGetHandleByIndex(idx)
        self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self._h, nv.NVML_CLOCK_SM)

    def _run(self):
        try:
            nv, h = self._nv, self._h
            names = {
                getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            while not self._stop.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
                time.sleep(0.002)
        except Exception as e:  # NVML missing: report that, do not fail the run
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def __enter__(self):
        try:
            self._open()  # NVML start-up takes longer than a short timed region: do it before
        except Exception as e:
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")
            return self
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(2)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def dist_setup(gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert world == gpus, f"--gpus {gpus} but WORLD_SIZE={world}: launch N>1 with torchrun"
    return world, rank, local


def max_over_ranks(ms, world):
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


# --------------------------------------------------------------------------- our arm
def make_layer(shard, dev):
    """The rank's slice of the layer: all heads of its batch rows, or some heads of one batch row."""
    from lookahead_keys_attention_b200 import Castle
    torch.manual_seed(0)
    full = Castle(CFG["dim"], heads=CFG["heads"], dim_head=CFG["dim_head"])
    hs = shard.h1 - shard.h0
    m = Castle(CFG["dim"], heads=hs, dim_head=CFG["dim_head"])
    d = CFG["dim_head"]
    with torch.no_grad():
        w = full.to_all_qkv.weight.view(6, CFG["heads"], d, CFG["dim"])[:, shard.h0:shard.h1]
        m.to_all_qkv.weight.copy_(w.reshape(6 * hs * d, CFG["dim"]))
        m.combine_heads.weight.copy_(full.combine_heads.weight[:, shard.h0 * d:shard.h1 * d])
    return m.to(dev).bfloat16()


def run_ours(args):
    world, rank, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    from lookahead_keys_attention_b200 import _lib, castle_attention_packed, check_status
    from lookahead_keys_attention_b200.sharding import partition
    lib = _lib.load()
    peaks = load_peaks()
    B, N, H, d, dim = (CFG[k] for k in ("batch", "seq_len", "heads", "dim_head", "dim"))
    weak = args.scaling == "weak"
    shard = partition(B, H, 1, 0) if weak else partition(B, H, world, rank)
    bs, hs = shard.b1 - shard.b0, shard.h1 - shard.h0
    layer = make_layer(shard, dev)
    g = torch.Generator().manual_seed(1)
    x_host = torch.randn(B, N, dim, generator=g).bfloat16()[shard.b0:shard.b1].contiguous().pin_memory()
    g_host = torch.randn(B, N, dim, generator=g).bfloat16()[shard.b0:shard.b1].contiguous().pin_memory()

    # ---- core arm: q/k/v resident in HBM, as views of the packed projection output
    with torch.no_grad():
        packed = layer.to_all_qkv(x_host.to(dev)).view(bs, N, 6, hs, d)
    packed.requires_grad_()
    gcore = torch.randn(bs, N, hs, d, device=dev, generator=torch.Generator(dev).manual_seed(2)).bfloat16().permute(0, 2, 1, 3)
    scale = d ** -0.5

    def core_step():
        packed.grad = None
        out = castle_attention_packed(packed, scale, False)
        out.backward(gcore)

    for _ in range(args.warmup):
        core_step()
    torch.cuda.synchronize()
    check_status()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    for row in ev:
        for e in row:
            e.record()  # torch creates the underlying cudaEvent_t lazily; the library records into it later
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    with ClockSampler(local) as clocks:
        e0.record()
        for s in range(args.steps):
            lib.castle_set_kernel_events(0, ev[s][0].cuda_event, ev[s][1].cuda_event)
            lib.castle_set_kernel_events(1, ev[s][2].cuda_event, ev[s][3].cuda_event)
            core_step()
        e1.record()
        barrier(world)
    lib.castle_set_kernel_events(0, None, None)
    lib.castle_set_kernel_events(1, None, None)
    check_status()
    ms_core = max_over_ranks(e0.elapsed_time(e1) / args.steps, world)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    bwd_ms = sum(e[2].elapsed_time(e[3]) for e in ev) / args.steps
    f_fwd, f_bwd = core_flops(B, H, N, d)
    if weak:
        f_fwd, f_bwd = f_fwd * world, f_bwd * world
    value = (f_fwd + f_bwd) / (ms_core * 1e-3) / 1e12
    rank_f_fwd, rank_f_bwd = core_flops(bs, hs, N, d)
    bwd_tflops = rank_f_bwd / (bwd_ms * 1e-3) / 1e12
    fwd_tflops = rank_f_fwd / (fwd_ms * 1e-3) / 1e12

    # ---- the final gather of the sharded path (untimed in `value`): every rank's core output to rank 0
    gather = None
    if world > 1 and not weak:
        from lookahead_keys_attention_b200.sharding import gather_heads
        with torch.no_grad():
            out_local = castle_attention_packed(packed.detach(), scale, False)
            gather_heads(out_local, shard, B, H)   # warm-up (NCCL sets its channels up on first use)
            barrier(world)
            ge0, ge1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ge0.record()
            full_out = gather_heads(out_local, shard, B, H)
            ge1.record()
            barrier(world)
            g_ms = max_over_ranks(ge0.elapsed_time(ge1), world)
            if rank == 0:
                ok = bool(torch.equal(full_out[shard.b0:shard.b1, shard.h0:shard.h1], out_local)) and \
                    bool(torch.isfinite(full_out.float()).all()) and tuple(full_out.shape) == (B, H, N, d)
                gather = {"ms": round(g_ms, 3), "bytes": full_out.numel() * full_out.element_size(), "checked": ok,
                          "what": "gather_heads: (batch, head) rectangles of the core output to rank 0 over NCCL"}
            del full_out, out_local

    # ---- end-to-end arm: the module called with host tensors
    group = None
    run_layer = layer
    if world > B and not weak:
        # Ranks that share a batch row split its heads for the attention core.  The projections around the
        # core are split by POSITIONS instead (full weights on every rank) and the tensors change hands by an
        # all-to-all inside the row's group before and after the core, so every rank uploads, projects and
        # downloads only its own positions and nothing is summed across ranks.
        import torch.distributed as dist
        from lookahead_keys_attention_b200.sharding import Shard, heads_to_rows, rows_to_heads
        per = world // B
        for b in range(B):
            grp = dist.new_group(list(range(b * per, (b + 1) * per)))
            if b == shard.b0:
                group = grp
        full = make_layer(Shard(shard.b0, shard.b1, 0, H), dev)
        n_r = N // per
        r0 = (rank % per) * n_r
        x_host = x_host[:, r0:r0 + n_r].contiguous().pin_memory()
        g_host = g_host[:, r0:r0 + n_r].contiguous().pin_memory()

        def run_layer(x):
            qkv = full.to_all_qkv(full.norm(x))
            packed_h = rows_to_heads(qkv.view(1, n_r, 6, H, d), group)            # every position, this rank's heads
            o = castle_attention_packed(packed_h, scale, False)                     # (1, H/per, N, d)
            return full.combine_heads(heads_to_rows(o, group))                     # this rank's positions

        layer = full   # its parameters are the ones whose gradients are cleared per step
    out_host = torch.empty_like(x_host).pin_memory()
    dx_host = torch.empty_like(x_host).pin_memory()

    # Host copies run on their own streams, double-buffered: the H2D copy of step s+1 and the D2H
    # copy of step s-1 overlap the compute of step s.  Every step still copies its own inputs in
    # from pinned host memory and its results (out, dx) back, inside the timed region.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    dbuf = [(torch.empty_like(x_host, device=dev), torch.empty_like(g_host, device=dev)) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_done = torch.cuda.Event()
    ev_out = [torch.cuda.Event() for _ in range(2)]
    hold = [None, None]  # results stay referenced until their D2H copy is known to be done (no record_stream:
    #                      it would make the caching allocator grow, and cudaMalloc, inside the timed region)

    def prefetch(slot):
        s_in.wait_event(ev_free[slot])
        with torch.cuda.stream(s_in):
            dbuf[slot][0].copy_(x_host, non_blocking=True)
            dbuf[slot][1].copy_(g_host, non_blocking=True)
            ev_in[slot].record(s_in)

    def e2e_run(n):
        for e in ev_free + ev_out:
            e.record(main)
        prefetch(0)
        for s_ in range(n):
            slot = s_ % 2
            if s_ + 1 < n:
                prefetch((s_ + 1) % 2)
            main.wait_event(ev_in[slot])
            main.wait_event(ev_out[slot])   # the copy that read hold[slot] two steps ago has finished
            hold[slot] = None
            x = dbuf[slot][0].detach().requires_grad_()
            for p_ in layer.parameters():
                p_.grad = None
            out = run_layer(x)
            out.backward(dbuf[slot][1])
            dx, o = x.grad, out.detach()
            hold[slot] = (o, dx)
            ev_free[slot].record(main)
            ev_done.record(main)
            s_out.wait_event(ev_done)
            with torch.cuda.stream(s_out):
                out_host.copy_(o, non_blocking=True)
                dx_host.copy_(dx, non_blocking=True)
                ev_out[slot].record(s_out)
        main.wait_stream(s_out)
        hold[0] = hold[1] = None

    if not args.no_e2e:
        e2e_run(args.warmup)
    barrier(world)
    e0.record()
    if not args.no_e2e:
        e2e_run(args.steps)
    e1.record()
    barrier(world)
    check_status()
    ms_e2e = max_over_ranks(max(e0.elapsed_time(e1), 1e-6) / args.steps, world)
    e2e_value = (f_fwd + f_bwd) / (ms_e2e * 1e-3) / 1e12

    line = {
        "metric": "castle_attn_fwd_bwd_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_core, 4), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"castle_attention_layer B={B} N={N} H={H} d_head={d} dim={dim}, forward+backward",
                   "sharding": f"batch x head rectangles, {bs}x{hs} pairs per GPU", "flops": "19*B*H*N^2*d algorithmic",
                   "l2": "inputs_exceed_l2 (q/k/v, grads and scratch of one step are > 126 MB)"},
        "frac_of_tensor_peak": round(value / (peaks["tflops"] * world), 4),
        "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": 2 * x_host.numel() * 2 * world,
                "d2h_bytes_per_step": 2 * out_host.numel() * 2 * world,
                "exchange": None if group is None else "positions <-> heads all-to-all inside each batch row's group, twice per pass"},
        "gpu_launches": 5 * args.steps,
        "kernels": {"fwd_main_ms": round(fwd_ms, 4), "fwd_main_tflops": round(fwd_tflops, 2),
                    "bwd_main_ms": round(bwd_ms, 4), "bwd_main_tflops": round(bwd_tflops, 2)},
        "roofline": {"kernel": "castle_bwd_kernel", "bound": "tensor", "achieved": round(bwd_tflops, 2),
                     "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": round(bwd_tflops / peaks["tflops"], 4),
                     "traffic": captured_traffic(f"bwd_d{d}_N{N}", bs * hs),
                     "traffic_source": "profiles/ncu_dram_traffic.txt (ncu capture of a smaller launch, scaled by batch*head pairs)",
                     "peak_source": f"{peaks['source']} bf16 burst"},
        "clocks": clocks.summary(),
    }
    if args.no_e2e:
        line["e2e"] = None
    if gather is not None:
        line["gather"] = gather
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(steps=2, warmup=1)
    if not args.no_decode:
        dec = run_decode(args, world, rank, dev, peaks)
        if rank == 0:
            line["decode"] = dec
    if not args.no_extra:
        c4 = run_cfg4(world, dev, peaks)
        if rank == 0:
            line["cfg4"] = c4
        if world == 1:
            line["cfg3"] = run_cfg3(dev)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


CFG4 = dict(batch=1, seq_len=16384, heads=32, dim_head=128, dim=4096, warmup=3, steps=5)
CFG3 = dict(layers=8, dim=512, heads=8, dim_head=64, batch=16, seq_len=1024, warmup=3, steps=5)


def run_cfg4(world, dev, peaks):
    """Long-context configuration (B=8, N=16384, H=32, d_head=128 over 8 GPUs): every rank runs ONE per-GPU
    slice (B=1, all 32 heads) of it, forward + backward of the core on the packed projection output."""
    from lookahead_keys_attention_b200 import _lib, castle_attention_packed, check_status, release_workspaces
    lib = _lib.load()
    c = CFG4
    B, N, H, d, dim = (c[k] for k in ("batch", "seq_len", "heads", "dim_head", "dim"))
    gen = torch.Generator(dev).manual_seed(11)
    with torch.no_grad():
        w = torch.empty(6 * H * d, dim, device=dev).uniform_(-dim ** -0.5, dim ** -0.5, generator=gen).bfloat16()
        x = torch.randn(B, N, dim, device=dev, generator=gen).bfloat16()
        packed = (x @ w.T).view(B, N, 6, H, d)
        del w, x
    packed.requires_grad_()
    g = torch.randn(B, N, H, d, device=dev, generator=gen).bfloat16().permute(0, 2, 1, 3)
    scale = d ** -0.5

    def step():
        packed.grad = None
        castle_attention_packed(packed, scale, False).backward(g)

    for _ in range(c["warmup"]):
        step()
    torch.cuda.synchronize()
    check_status()
    n = c["steps"]
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n)]
    for row in ev:
        for e in row:
            e.record()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    e0.record()
    for s_ in range(n):
        lib.castle_set_kernel_events(0, ev[s_][0].cuda_event, ev[s_][1].cuda_event)
        lib.castle_set_kernel_events(1, ev[s_][2].cuda_event, ev[s_][3].cuda_event)
        step()
    e1.record()
    barrier(world)
    lib.castle_set_kernel_events(0, None, None)
    lib.castle_set_kernel_events(1, None, None)
    check_status()
    ms = max_over_ranks(e0.elapsed_time(e1) / n, world)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / n
    bwd_ms = sum(e[2].elapsed_time(e[3]) for e in ev) / n
    f_fwd, f_bwd = core_flops(B, H, N, d)
    tf = (f_fwd + f_bwd) * world / (ms * 1e-3) / 1e12
    nblk = -(-N // 128)
    del packed, g
    release_workspaces()
    torch.cuda.empty_cache()
    return {"metric": "castle_attn_fwd_bwd_tflops", "value": round(tf, 2), "unit": "TFLOP/s", "ms_per_step": round(ms, 3),
            "steps": n, "warmup": c["warmup"],
            "config": {"workload": f"long-context slice per GPU: B={B} N={N} H={H} d_head={d} (1/8 of B=8), forward+backward of the core",
                       "slices": world},
            "frac_of_tensor_peak": round(tf / (peaks["tflops"] * world), 4),
            "kernels": {"fwd_main_ms": round(fwd_ms, 3), "fwd_main_tflops": round(f_fwd / (fwd_ms * 1e-3) / 1e12, 2),
                        "bwd_main_ms": round(bwd_ms, 3), "bwd_main_tflops": round(f_bwd / (bwd_ms * 1e-3) / 1e12, 2)},
            "roofline": {"kernel": "castle_bwd128_kv_kernel + castle_bwd128_la_kernel", "bound": "tensor",
                         "achieved": round(f_bwd / (bwd_ms * 1e-3) / 1e12, 2), "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": round(f_bwd / (bwd_ms * 1e-3) / 1e12 / peaks["tflops"], 4),
                         "traffic": captured_traffic("bwd_d128", B * H * nblk * (nblk + 1) // 2),
                         "traffic_source": "profiles/ncu_dram_traffic.txt (ncu capture of a smaller launch pair, scaled by (query block, key block) steps)",
                         "peak_source": f"{peaks['source']} bf16 burst"}}


class ByteLM(torch.nn.Module):
    """The model shape of the reference's training script (train_triton.py:73-175 there): byte embedding,
    layers of [Castle(prenorm) + residual, RMSNorm -> 4x GELU FFN + residual], final RMSNorm, logits."""

    def __init__(self, layers, dim, heads, dim_head):
        from torch import nn
        from lookahead_keys_attention_b200 import Castle
        super().__init__()
        self.emb = nn.Embedding(256, dim)
        self.attn = nn.ModuleList([Castle(dim, heads=heads, dim_head=dim_head, prenorm=True) for _ in range(layers)])
        self.ff = nn.ModuleList([nn.Sequential(nn.RMSNorm(dim), nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))
                                 for _ in range(layers)])
        self.norm = nn.RMSNorm(dim)
        self.logits = nn.Linear(dim, 256, bias=False)

    def forward(self, ids):
        x, y = ids[:, :-1], ids[:, 1:]
        h = self.emb(x)
        for a, f in zip(self.attn, self.ff):
            h = a(h) + h
            h = f(h) + h
        return torch.nn.functional.cross_entropy(self.logits(self.norm(h)).float().flatten(0, 1), y.flatten())


def cfg3_graph_step(lm, ids, c):
    """The same training step captured once in a CUDA graph and replayed: the eager step is bound by ~400 small
    launches, not by the GPU.  Returns its own ms per step and tokens/s (or why the capture was not possible)."""
    from lookahead_keys_attention_b200 import check_status
    try:
        opt = torch.optim.Adam(lm.parameters(), lr=1e-4, capturable=True)
        static_loss = [None]

        def step():
            opt.zero_grad(set_to_none=True)
            loss = lm(ids)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(lm.parameters(), 0.5)
            opt.step()
            static_loss[0] = loss.detach()

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        first = float(static_loss[0])
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        for _ in range(c["warmup"]):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(c["steps"]):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        check_status()
        ms = e0.elapsed_time(e1) / c["steps"]
        return {"ms_per_step": round(ms, 3), "tokens_per_s": round(c["batch"] * c["seq_len"] / (ms * 1e-3), 1),
                "loss_first_last": [round(first, 4), round(float(static_loss[0]), 4)]}
    except Exception as e:  # a failed capture must not take the bench line with it
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def run_cfg3(dev):
    """8-layer byte LM, bf16 training step (forward, backward, clip, Adam) on batch 16 x 1024 uniform bytes."""
    from lookahead_keys_attention_b200 import check_status
    c = CFG3
    torch.manual_seed(5)
    lm = ByteLM(c["layers"], c["dim"], c["heads"], c["dim_head"]).to(dev).bfloat16()
    opt = torch.optim.Adam(lm.parameters(), lr=1e-4)
    ids = torch.randint(0, 256, (c["batch"], c["seq_len"] + 1), device=dev)
    losses = []

    def step():
        opt.zero_grad(set_to_none=True)
        loss = lm(ids)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(lm.parameters(), 0.5)
        opt.step()
        losses.append(loss.detach())

    for _ in range(c["warmup"]):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(c["steps"]):
        step()
    e1.record()
    torch.cuda.synchronize()
    check_status()
    ms = e0.elapsed_time(e1) / c["steps"]
    graph = cfg3_graph_step(lm, ids, c)
    return {"metric": "lm_train_tokens_per_s", "value": round(c["batch"] * c["seq_len"] / (ms * 1e-3), 1), "unit": "tokens/s",
            "ms_per_step": round(ms, 3), "steps": c["steps"], "warmup": c["warmup"],
            "loss_first_last": [round(float(losses[0]), 4), round(float(losses[-1]), 4)],
            "cuda_graph": graph,
            "config": {"workload": f"{c['layers']}-layer byte LM, dim {c['dim']}, {c['heads']} heads x {c['dim_head']}, pre-RMSNorm, 4x GELU FFN, "
                                   f"batch {c['batch']} x {c['seq_len']} uniform bytes, bf16, Adam, clip 0.5 (one step = fwd + bwd + optimizer)"}}


def run_decode(args, world, rank, dev, peaks):
    """Cached decode: B=64 (split by batch over ranks), prefix prefilled through the parallel pass."""
    from lookahead_keys_attention_b200 import Castle, _lib, check_status
    lib = _lib.load()
    c = DECODE_CFG
    bs = c["batch"] // world
    torch.manual_seed(3)
    m = Castle(c["dim"], heads=c["heads"], dim_head=c["dim_head"], cache_headroom=c["steps"] + 8).to(dev).bfloat16()
    gen = torch.Generator(dev).manual_seed(4 + rank)
    steps, warm = c["steps"], 3
    with torch.no_grad():
        # prefill in batch slices so the packed projection of the prefix stays a few GB
        caches = []
        for b0 in range(0, bs, 8):
            xb = torch.randn(min(8, bs - b0), c["prefix"], c["dim"], device=dev, generator=gen).bfloat16()
            _, cb = m(xb, return_next_cache=True)
            caches.append(cb)
            del xb
        # one capacity buffer per cache for the whole rank-local batch
        cap = c["prefix"] + steps + warm + 8
        bufs = [torch.empty(bs, c["heads"], cap, c["dim_head"], dtype=torch.bfloat16, device=dev) for _ in range(4)]
        for i in range(4):
            b0 = 0
            for cb in caches:
                n = cb[i].shape[0]
                bufs[i][b0:b0 + n, :, :c["prefix"]].copy_(cb[i])
                b0 += n
        del caches
        from lookahead_keys_attention_b200 import cache_from_buffers
        cache = cache_from_buffers(*bufs, length=c["prefix"])   # the module appends to these buffers in place
        xs = torch.randn(steps + warm, bs, 1, c["dim"], device=dev, generator=gen).bfloat16()
        for s in range(warm):
            _, cache = m(xs[s], cache=cache)
        torch.cuda.synchronize()
        check_status()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(steps)]
        for a, b in ev:
            a.record(); b.record()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier(world)
        e0.record()
        for s in range(steps):
            lib.castle_set_kernel_events(2, ev[s][0].cuda_event, ev[s][1].cuda_event)
            _, cache = m(xs[warm + s], cache=cache)
        e1.record()
        barrier(world)
        lib.castle_set_kernel_events(2, None, None)
        check_status()
    ms = max_over_ranks(e0.elapsed_time(e1) / steps, world)
    kms = sum(a.elapsed_time(b) for a, b in ev) / steps
    t_mean = c["prefix"] + warm + (steps - 1) / 2
    alg_bytes = bs * c["heads"] * 5 * t_mean * c["dim_head"] * 2
    gbs = alg_bytes / (kms * 1e-3) / 1e9
    return {"metric": "decode_tokens_per_s", "value": round(c["batch"] / (ms * 1e-3), 1), "unit": "tokens/s",
            "ms_per_step": round(ms, 4), "kernel_ms": round(kms, 4),
            "config": {"workload": f"cached decode B={c['batch']} H={c['heads']} d_head={c['dim_head']} prefix={c['prefix']} steps={steps}",
                       "per_gpu_batch": bs},
            "roofline": {"kernel": "castle_decode_ring_kernel", "bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm"],
                         "unit": "GB/s", "frac": round(gbs / peaks["hbm"], 4),
                         "traffic": captured_traffic(f"decode_d{c['dim_head']}", alg_bytes),
                         "algorithmic_bytes_per_launch": int(alg_bytes), "peak_source": peaks["source"]}}


# --------------------------------------------------------------------------- CPU reference arm
CPU_SAMPLE_HEADS = 2


def cpu_sample_time(steps, warmup):
    """Forward + backward of the reference's own PyTorch path on the host cores, on a bounded sample
    of the workload: 1 batch row x 2 heads at the full N=4096, d=64, bf16.

    When the staged copy of the reference is present (oracle/_ref, made by oracle/make_ref.py) the
    thing timed is the reference's `Castle(use_triton=False)` module, forward + AUTOGRAD backward
    (lookahead_keys_attention.py:132-164), projections included; otherwise the oracle port (same
    arithmetic, closed-form backward).  Either way the flops credited are the algorithmic 19u of the
    sample's attention core."""
    from oracle import make_ref
    N, d, hs, dim = CFG["seq_len"], CFG["dim_head"], CPU_SAMPLE_HEADS, CFG["dim"]
    torch.set_num_threads(os.cpu_count() or 1)   # launchers set OMP_NUM_THREADS=1; the baseline may use every core
    torch.manual_seed(0)
    if make_ref.available():
        RefCastle = make_ref.load_reference()
        m = RefCastle(dim, heads=hs, dim_head=d, use_triton=False).bfloat16()
        x = torch.randn(1, N, dim).bfloat16().requires_grad_()
        g = torch.randn(1, N, dim).bfloat16()

        def step():
            x.grad = None
            m.zero_grad(set_to_none=True)
            m(x).backward(g)

        kind = "reference"
        what = "the reference's Castle(use_triton=False) from oracle/_ref, forward + autograd backward, projections included"
    else:
        from oracle import castle_oracle as O
        t = [(torch.randn(1, hs, N, d) * 3 ** -0.5).bfloat16() for _ in range(6)]
        g = torch.randn(1, hs, N, d).bfloat16()
        scale = d ** -0.5

        def step():
            O.castle_parallel(*t, scale)
            O.castle_parallel_bwd(*t, scale, g)

        kind = "port"
        what = "oracle port (oracle/_ref not staged), forward + closed-form backward of the core"
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    f_fwd, f_bwd = core_flops(1, hs, N, d)
    sample = f"1 batch row x {hs} heads of the workload (N={N}, d={d}, dim={dim}), bf16: {what}"
    return dt, (f_fwd + f_bwd) / dt / 1e12, sample, kind


def cpu_baseline(steps, warmup):
    dt, tf, sample, kind = cpu_sample_time(steps, warmup)
    return {"value": round(tf, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": sample, "s_per_sample": round(dt, 3)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = args.steps, max(args.warmup, 1)
    dt, tf, sample, kind = cpu_sample_time(steps, warm)
    B, N, H, d, dim = (CFG[k] for k in ("batch", "seq_len", "heads", "dim_head", "dim"))
    line = {
        "impl": "reference", "metric": "castle_attn_fwd_bwd_tflops", "value": round(tf, 5), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": round(dt * 1e3, 2),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"castle_attention_layer B={B} N={N} H={H} d_head={d} dim={dim}, forward+backward",
                   "sample_per_step": f"1 batch row x {CPU_SAMPLE_HEADS} heads of the {B}x{H} (batch, head) pairs, at the full N",
                   "flops": "19*B*H*N^2*d algorithmic, of the sample"},
        "cpu_baseline": {"value": round(tf, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample},
        "e2e": {"value": round(tf, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong (default): the fixed B=4,H=16 problem is split over the GPUs, as the benchmark "
                         "configuration says; weak: every GPU runs the whole problem (global batch 4*N)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end arm (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="skip the long-context slice and the LM step (profiling runs)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline (profiling runs)")
    ap.add_argument("--batch", type=int, default=None, help="override B (smaller case of the same workload, for ncu)")
    ap.add_argument("--seq-len", type=int, default=None, help="override N (for ncu captures)")
    ap.add_argument("--heads", type=int, default=None, help="override H (other configurations of the same layer)")
    ap.add_argument("--dim-head", type=int, default=None, help="override d_head (64 or 128)")
    ap.add_argument("--dim", type=int, default=None, help="override the model width")
    ap.add_argument("--decode-steps", type=int, default=None, help="override the number of decode steps (for ncu)")
    ap.add_argument("--decode-batch", type=int, default=None, help="override the decode batch (for ncu)")
    args = ap.parse_args()
    if args.batch:
        CFG["batch"] = args.batch
    if args.seq_len:
        CFG["seq_len"] = args.seq_len
    if args.heads:
        CFG["heads"] = args.heads
    if args.dim_head:
        CFG["dim_head"] = args.dim_head
    if args.dim:
        CFG["dim"] = args.dim
    if args.decode_steps:
        DECODE_CFG["steps"] = args.decode_steps
    if args.decode_batch:
        DECODE_CFG["batch"] = args.decode_batch
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
