"""GPU: the module inside a byte-level decoder LM (the model shape of the reference's training script,
train_triton.py:73-175 there: token embedding, N x [Castle(prenorm) + residual, RMSNorm -> 4x GELU
FFN + residual], final RMSNorm, logits, cross-entropy on next-byte targets), one bf16 training step
on synthetic uniform bytes.  Parity: the same stack with the attention core replaced by the CPU
oracle (fp32 on the same bf16-rounded weights); then the full-size step of the benchmark
configuration (8 layers, dim 512, 8 heads x 64, batch 16 x 1024 tokens) runs and learns."""
import pytest
import torch
from torch import nn

from oracle import castle_oracle as O

pytestmark = pytest.mark.gpu


class ByteLM(nn.Module):
    def __init__(self, layers, dim, heads, dim_head, castle_cls):
        super().__init__()
        self.emb = nn.Embedding(256, dim)
        self.attn = nn.ModuleList([castle_cls(dim, heads=heads, dim_head=dim_head, prenorm=True) for _ in range(layers)])
        self.ff = nn.ModuleList([nn.Sequential(nn.RMSNorm(dim), nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))
                                 for _ in range(layers)])
        self.norm = nn.RMSNorm(dim)
        self.logits = nn.Linear(dim, 256, bias=False)

    def logits_with_cache(self, ids, caches=None):
        """Per-layer cache list, the way the reference's sampling loop threads it (train_triton.py:113-139 there)."""
        h = self.emb(ids)
        new = []
        for i, (a, f) in enumerate(zip(self.attn, self.ff)):
            o, c = a(h, cache=None if caches is None else caches[i], return_next_cache=True)
            new.append(c)
            h = o + h
            h = f(h) + h
        return self.logits(self.norm(h)), new

    def forward(self, ids):
        x, y = ids[:, :-1], ids[:, 1:]
        h = self.emb(x)
        for a, f in zip(self.attn, self.ff):
            h = a(h) + h
            h = f(h) + h
        return nn.functional.cross_entropy(self.logits(self.norm(h)).float().flatten(0, 1), y.flatten())


class OracleCastle(nn.Module):
    """Same parameters and state-dict keys as Castle, core evaluated by the CPU oracle."""

    def __init__(self, dim, heads=8, dim_head=64, prenorm=False):
        super().__init__()
        self.heads, self.dim_head = heads, dim_head
        self.norm = nn.RMSNorm(dim) if prenorm else nn.Identity()
        self.to_all_qkv = nn.Linear(dim, heads * dim_head * 6, bias=False)
        self.combine_heads = nn.Linear(heads * dim_head, dim, bias=False)

    def forward(self, x):
        nw = self.norm.weight if isinstance(self.norm, nn.RMSNorm) else None
        return O.castle_module_forward(x, self.to_all_qkv.weight, self.combine_heads.weight, self.heads, self.dim_head,
                                       norm_weight=nw)


def test_lm_step_matches_oracle_stack():
    from lookahead_keys_attention_b200 import Castle
    torch.manual_seed(0)
    ours = ByteLM(2, 128, 2, 64, Castle).cuda().bfloat16()
    ref = ByteLM(2, 128, 2, 64, OracleCastle)
    ref.load_state_dict({k: v.float().cpu() for k, v in ours.state_dict().items()})  # same keys, bf16-rounded values
    ids = torch.randint(0, 256, (2, 257))
    loss = ours(ids.cuda())
    loss.backward()
    loss_ref = ref(ids)
    loss_ref.backward()
    assert abs(loss.item() - loss_ref.item()) < 2e-2, (loss.item(), loss_ref.item())
    gn = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in ours.parameters())).item()
    gn_ref = torch.sqrt(sum((p.grad ** 2).sum() for p in ref.parameters())).item()
    assert abs(gn - gn_ref) <= 3e-2 * gn_ref, (gn, gn_ref)
    for (n, p), (_, q) in zip(ours.named_parameters(), ref.named_parameters()):
        rel = ((p.grad.float().cpu() - q.grad).norm() / (q.grad.norm() + 1e-6)).item()
        assert rel < 5e-2, f"{n}: rel-F {rel:.3e}"


def test_lm_step_full_depth_matches_oracle_stack():
    """The benchmark model at its full depth and width (8 layers, dim 512, 8 heads x 64, 1024 tokens) on a
    quarter of its batch: loss and gradient norm of one bf16 step against the same stack with the attention
    core evaluated by the CPU oracle in fp32 on the same bf16-rounded weights."""
    from lookahead_keys_attention_b200 import Castle, check_status
    torch.manual_seed(3)
    ours = ByteLM(8, 512, 8, 64, Castle).cuda().bfloat16()
    ref = ByteLM(8, 512, 8, 64, OracleCastle)
    ref.load_state_dict({k: v.float().cpu() for k, v in ours.state_dict().items()})
    ids = torch.randint(0, 256, (4, 1025))
    loss = ours(ids.cuda())
    loss.backward()
    check_status()
    loss_ref = ref(ids)
    loss_ref.backward()
    assert abs(loss.item() - loss_ref.item()) < 3e-2, (loss.item(), loss_ref.item())
    gn = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in ours.parameters())).item()
    gn_ref = torch.sqrt(sum((p.grad ** 2).sum() for p in ref.parameters())).item()
    assert abs(gn - gn_ref) <= 5e-2 * gn_ref, (gn, gn_ref)
    # the attention projections of the first and the last layer, where errors of the whole stack show
    for name in ("attn.0.to_all_qkv.weight", "attn.7.to_all_qkv.weight", "attn.7.combine_heads.weight"):
        a = dict(ours.named_parameters())[name].grad.float().cpu()
        b = dict(ref.named_parameters())[name].grad
        rel = ((a - b).norm() / (b.norm() + 1e-6)).item()
        assert rel < 8e-2, f"{name}: rel-F {rel:.3e}"


def test_lm_training_steps_full_size():
    from lookahead_keys_attention_b200 import Castle, check_status
    torch.manual_seed(0)
    lm = ByteLM(8, 512, 8, 64, Castle).cuda().bfloat16()
    opt = torch.optim.Adam(lm.parameters(), lr=1e-3)
    ids = torch.randint(0, 256, (16, 1025), device="cuda")
    losses = []
    for _ in range(4):
        opt.zero_grad(set_to_none=True)
        loss = lm(ids)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(lm.parameters(), 0.5)
        opt.step()
        losses.append(loss.item())
    check_status()
    assert all(torch.isfinite(torch.tensor(losses))) and 4.5 < losses[0] < 7.0  # ln(256) = 5.55 at init
    assert losses[-1] < losses[0], losses  # the same batch is fitted a little better each step


@torch.no_grad()
def test_lm_prompt_then_cached_decode_matches_teacher_forcing():
    """Feed a prompt once (parallel pass, caches returned), then one token at a time with the per-layer cache
    list; the logits must equal those of a single parallel pass over the whole sequence."""
    from lookahead_keys_attention_b200 import Castle, check_status
    torch.manual_seed(1)
    lm = ByteLM(3, 128, 2, 64, Castle).cuda()
    ids = torch.randint(0, 256, (2, 48), device="cuda")
    full, _ = lm.logits_with_cache(ids)
    logits, caches = lm.logits_with_cache(ids[:, :32])
    outs = [logits]
    for t in range(32, 48):
        logits, caches = lm.logits_with_cache(ids[:, t:t + 1], caches)
        outs.append(logits)
    check_status()
    assert torch.allclose(torch.cat(outs, 1), full, atol=2e-3)
