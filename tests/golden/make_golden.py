"""Generate the golden vectors under tests/golden/ from the REAL reference.

Run once, in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/lookahead-keys-attention

The reference's module imports `rotary_embedding_torch`, which may be absent;
a placeholder module is registered for the import only (rotary is never
enabled in any vector below).  Everything recorded is the reference's own
output: module outputs, caches, and autograd gradients of its PyTorch path
(`use_triton=False`).  Inputs are rebuilt from the seeds stored in each file,
so the fixtures stay small; the fp64 core vectors are stored rounded to fp32.
"""
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference(path):
    try:
        import rotary_embedding_torch  # noqa: F401
    except ImportError:
        stub = types.ModuleType("rotary_embedding_torch")
        stub.RotaryEmbedding = object
        sys.modules["rotary_embedding_torch"] = stub
    sys.path.insert(0, str(path))
    from lookahead_keys_attention.lookahead_keys_attention import Castle
    return Castle


def module_case(Castle, name, dim, heads, dim_head, prenorm, b, n, split, seed, dtype=torch.float32, stride=1):
    """parallel output (+grads), prefill cache at `split`, then cached single-token steps."""
    torch.manual_seed(seed)
    m = Castle(dim, heads=heads, dim_head=dim_head, use_triton=False, prenorm=prenorm).to(dtype)
    if prenorm:
        with torch.no_grad():
            m.norm.weight.uniform_(0.5, 1.5)
    x = torch.randn(b, n, dim, dtype=dtype)
    g = torch.randn(b, n, dim, dtype=dtype)
    xr = x.clone().requires_grad_()
    out = m(xr)
    out.backward(g)
    rec = {
        "meta": np.array([dim, heads, dim_head, int(prenorm), b, n, split, seed, stride]),
        "out": out.detach()[:, ::stride].numpy(),
        "dx": xr.grad[:, ::stride].numpy(),
        "dw_qkv_sum_abs": m.to_all_qkv.weight.grad.abs().sum().numpy(),
        "dw_qkv_sample": m.to_all_qkv.weight.grad[::37, ::11].numpy(),
        "dw_out_sample": m.combine_heads.weight.grad[::11, ::13].numpy(),
    }
    with torch.no_grad():
        pre, cache = m(x[:, :split], return_next_cache=True)
        rec["prefill_U"] = cache.U.numpy()
        steps = []
        for t in range(split, n):
            o, cache = m(x[:, t:t + 1], cache=cache, return_next_cache=True)
            steps.append(o)
        rec["seq_out"] = torch.cat([pre] + steps, dim=1)[:, ::stride].numpy()
        rec["final_U"] = cache.U[:, :, ::stride].numpy()
        rec["final_qu"] = cache.qu_cache[:, :, ::stride].numpy()
    np.savez_compressed(HERE / f"{name}.npz", **rec)
    print(name, {k: v.shape for k, v in rec.items()})


def core_case(Castle, name, b, h, n, d, seed):
    """Core tensors through the reference's own code: a Castle whose projections are
    identities exposes out, U and the six input gradients of the attention core."""
    torch.manual_seed(seed)
    m = Castle(6 * h * d, heads=h, dim_head=d, use_triton=False).double()
    with torch.no_grad():
        m.to_all_qkv.weight.copy_(torch.eye(6 * h * d, dtype=torch.double))
    m.combine_heads = torch.nn.Identity()
    packed = torch.randn(b, n, 6 * h * d, dtype=torch.double)
    g = torch.randn(b, n, h * d, dtype=torch.double)
    pr = packed.clone().requires_grad_()
    out, cache = m(pr, return_next_cache=True)
    out.backward(g)
    rec = {
        "meta": np.array([b, h, n, d, seed]),
        "out": out.detach().float().numpy(), "U": cache.U.detach().float().numpy(),
        "dpacked": pr.grad.float().numpy(),
    }
    np.savez_compressed(HERE / f"{name}.npz", **rec)
    print(name, {k: v.shape for k, v in rec.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to a checkout of lookahead-keys-attention>")
    Castle = load_reference(sys.argv[1])
    # shapes of the reference's own tests (tests/test_lookahead.py:18-23, 153-157, 75-79)
    module_case(Castle, "module_d16", 32, 2, 16, False, 2, 16, 8, 0)
    module_case(Castle, "module_d16_prenorm", 32, 2, 16, True, 2, 16, 8, 1)
    module_case(Castle, "module_d32", 64, 2, 32, False, 2, 32, 16, 2)
    module_case(Castle, "module_d64_n256", 128, 2, 64, True, 2, 256, 250, 3, stride=8)
    # README contract shape: Castle(512, heads=8, dim_head=64), x (2,128,512)
    module_case(Castle, "module_readme", 512, 8, 64, False, 2, 128, 120, 0, stride=16)
    core_case(Castle, "core_n40_d16", 1, 2, 40, 16, 4)
    core_case(Castle, "core_n200_d64", 1, 1, 200, 64, 5)
    core_case(Castle, "core_n130_d128", 1, 1, 130, 128, 6)
