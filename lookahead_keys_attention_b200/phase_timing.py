"""Developer aid: per-phase cycle counts of the parallel kernels.

Builds a DEBUG copy of the library with -DCASTLE_PHASE_TIMING (thread 0 of CTA (0,0) stores
clock64() at every phase boundary of its first eight tile steps behind the workspace), runs one
forward and a few backward passes on random inputs and prints the cycles each phase took.

    python -m lookahead_keys_attention_b200.phase_timing [B H N [d]] [-DMACRO ...]

The shipped library is built without the flag; this never touches it.
"""
import ctypes
import subprocess
import sys
import tempfile
from pathlib import Path

import torch

from . import _lib as L

PHASES = ["wait for Qc/Vu/Ku", "MMA Z", "gate A", "MMA peel, T", "masked T, Wb", "MMA Su", "penalty, silu'",
          "MMA Sc", "P", "MMA dvc, dP", "dS, dSu", "MMA dA (+dkc, X)", "dZ", "MMA G, dT", "masked dT",
          "issue X3, dqu, X2, X (3 commits)", "wait for the last commit", "stage dqc, issue its reduce", "-",
          "end barrier"]


KV_PHASES = ["wait for Qu, Ku, Vu, Qc (fetched in the step before)", "MMA Z", "gate A (+ drain wait of the dqc reduce)",
             "MMA peel, T", "masked T, Wb", "MMA Su", "penalty", "MMA Sc", "P", "MMA dvc, dP (+ wait Vc, dO)", "dS, dSu",
             "MMA dT (+ dkc behind)", "masked dT", "MMA dqc (3 commits, + wait Vu)", "stage dqc, issue reduces, end barrier"]

LA_PHASES = ["(issuing lanes refill the dku staging panels with Vu, Qc)", "wait for Qu, Ku, dO, Vc (fetched in the step before)",
             "MMA Z, dP", "gate A", "MMA peel, T", "masked T, Wb", "MMA Su", "penalty", "MMA Sc (+ wait Kc)",
             "P, dS, dSu", "MMA dA, G, dT", "dZ, masked dT", "MMA dvu, dqu part (+ wait Ku)",
             "stage dvu, dqu; issue reduces", "MMA dku (+ wait Qu, dvu reduce drained)", "stage dku, Gb; issue reduce"]

FWD_PHASES = ["MMA Z", "gate A", "MMA W update, T", "masked T", "MMA Su", "penalty, Wb", "MMA Sc", "soft-max, P",
              "MMA P.Vc", "partial store, end barrier"]


def main():
    extra = [a for a in sys.argv[1:] if a.startswith("-D")]   # e.g. -DCASTLE_TIMING_SKIP_REDUCE (wrong results, timing only)
    sys.argv = [a for a in sys.argv if not a.startswith("-D")]
    B, H, N = (int(a) for a in sys.argv[1:4]) if len(sys.argv) >= 4 else (4, 16, 4096)
    d = int(sys.argv[4]) if len(sys.argv) >= 5 else 64
    out = Path(tempfile.mkdtemp()) / "libcastle_timing.so"
    srcs = [str(L.CSRC / f) for f in ("api.cu", "fwd.cu", "bwd.cu", "bwd128.cu")]
    subprocess.run([L._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared", "-Xcompiler",
                    "-fPIC", "-DCASTLE_PHASE_TIMING", "-o", str(out)] + extra + srcs, check=True)
    lib = ctypes.CDLL(str(out))
    for name in ("castle_fwd", "castle_bwd", "castle_fwd_workspace_bytes", "castle_bwd_workspace_bytes"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = L._SIGNATURES[name]
    dev = "cuda"
    packed = (torch.randn(B, N, 6, H, d, device=dev) * 3 ** -0.5).bfloat16()
    qu, ku, vu, qc, kc, vc = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(6))
    o = torch.empty(B, N, H, d, device=dev, dtype=torch.bfloat16).permute(0, 2, 1, 3)
    do = torch.randn(B, N, H, d, device=dev).bfloat16().permute(0, 2, 1, 3)
    lse = torch.empty(B, H, N, device=dev)
    wst = torch.empty(B, H, N, d, device=dev)
    gp = torch.empty(B, N, 6, H, d, device=dev, dtype=torch.bfloat16)
    g = [gp[:, :, i].permute(0, 2, 1, 3) for i in range(6)]
    prob = L.CastleProblem(B, H, N, d, L.BF16, d ** -0.5)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    desc = lambda t: L.CastleTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    ref = lambda ts: [ctypes.byref(desc(t)) for t in ts]
    need_f = lib.castle_fwd_workspace_bytes(ctypes.byref(prob))
    wsf = torch.zeros(need_f + 4096, dtype=torch.uint8, device=dev)
    keep = [desc(t) for t in (qc, kc, vc, qu, ku, vu, o)]
    rc = lib.castle_fwd(ctypes.byref(prob), *[ctypes.byref(x) for x in keep], lse.data_ptr(), None, 0, wst.data_ptr(),
                        wsf.data_ptr(), wsf.numel(), st.data_ptr(), None)
    assert rc == 0, lib.castle_last_error()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        lib.castle_fwd(ctypes.byref(prob), *[ctypes.byref(x) for x in keep], lse.data_ptr(), None, 0, wst.data_ptr(),
                       wsf.data_ptr(), wsf.numel(), st.data_ptr(), None)
    e1.record()
    torch.cuda.synchronize()
    print(f"castle_fwd (both launches, timing build {' '.join(extra)}): {e0.elapsed_time(e1) / 5:.3f} ms per call")
    if d == 64:
        tf = wsf[need_f:need_f + 8 * 16 * 8].view(torch.int64).cpu().view(8, 16)[1:7, :11]
        df = (tf[:, 1:] - tf[:, :-1]).double().mean(0)
        print(f"castle_fwd_kernel_d64<bf16>  B={B} H={H} N={N}: cycles per phase, CTA (0,0), mean of tile steps 1-6")
        for name, c in zip(FWD_PHASES, df.tolist()):
            print(f"  {name:24s} {c:8.0f}")
        print(f"  {'total':24s} {df.sum().item():8.0f}")
    need = lib.castle_bwd_workspace_bytes(ctypes.byref(prob))
    ws = torch.zeros(need + 8192, dtype=torch.uint8, device=dev)
    a = [desc(t) for t in (qc, kc, vc, qu, ku, vu, o, do)]
    gr = [desc(t) for t in (g[3], g[4], g[5], g[0], g[1], g[2])]
    for _ in range(3):
        rc = lib.castle_bwd(ctypes.byref(prob), *[ctypes.byref(x) for x in a], lse.data_ptr(), wst.data_ptr(),
                            *[ctypes.byref(x) for x in gr], ws.data_ptr(), ws.numel(), st.data_ptr(), None)
        assert rc == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        lib.castle_bwd(ctypes.byref(prob), *[ctypes.byref(x) for x in a], lse.data_ptr(), wst.data_ptr(),
                       *[ctypes.byref(x) for x in gr], ws.data_ptr(), ws.numel(), st.data_ptr(), None)
    e1.record()
    torch.cuda.synchronize()
    print(f"castle_bwd (all four launches, timing build {' '.join(extra)}): {e0.elapsed_time(e1) / 5:.3f} ms per call")
    if d == 128:
        raw = ws[need:need + 8 * 32 * 8].view(torch.int64).cpu().view(8, 32)[1:7, :16]
        dt = (raw[:, 1:] - raw[:, :-1]).double().mean(0)
        print(f"castle_bwd128_kv_kernel<bf16>  B={B} H={H} N={N}: cycles per phase, CTA (0,0), mean of tile steps 1-6")
        for name, c in zip(KV_PHASES, dt.tolist()):
            print(f"  {name:44s} {c:8.0f}")
        print(f"  {'total':44s} {dt.sum().item():8.0f}")
        raw = ws[need + 2048:need + 2048 + 8 * 32 * 8].view(torch.int64).cpu().view(8, 32)[1:7, :17]
        dt = (raw[:, 1:] - raw[:, :-1]).double().mean(0)
        print(f"castle_bwd128_la_kernel<bf16>  B={B} H={H} N={N}: cycles per phase, CTA (0,0), mean of tile steps 1-6")
        for name, c in zip(LA_PHASES, dt.tolist()):
            print(f"  {name:44s} {c:8.0f}")
        print(f"  {'total':44s} {dt.sum().item():8.0f}")
        return
    raw = ws[need:need + 8 * 32 * 8].view(torch.int64).cpu().view(8, 32)[1:7]
    print("  within 'MMA peel, T': wait for Qc/Vu %.0f, products %.0f, group barrier (reduce drain) %.0f" % (
        (raw[:, 21] - raw[:, 3]).double().mean(), (raw[:, 22] - raw[:, 21]).double().mean(),
        (raw[:, 4] - raw[:, 22]).double().mean()))
    t = raw[:, :21]   # steps 1..6 of CTA (0,0)
    dt = (t[:, 1:] - t[:, :-1]).double().mean(0)
    print(f"castle_bwd_kernel<bf16,64>  B={B} H={H} N={N}: cycles per phase, CTA (0,0), mean of tile steps 1-6")
    for name, c in zip(PHASES, dt.tolist()):
        print(f"  {name:24s} {c:8.0f}")
    mma = sum(c for n, c in zip(PHASES, dt.tolist()) if n.startswith("MMA"))
    print(f"  {'total':24s} {dt.sum().item():8.0f}   (MMA phases {mma:.0f}, elementwise and waits {dt.sum().item() - mma:.0f})")


if __name__ == "__main__":
    main()
