"""GPU: the failure path of the kernels' bounded waits, made to run WITHOUT faulting the device.

Every mbarrier wait in the kernels polls a bounded number of times; when the polls run out the
CTA raises an abort flag, every later wait returns at once, the kernel frees its tensor memory
and ORs CASTLE_STATUS_WAIT_TIMEOUT into the status word the host reads.  The self-test kernel
walks exactly that path on a barrier nothing ever arrives on, with a small poll limit, and
returns normally.  The test then checks that the host side raises, clears the word, and that
the next ordinary forward pass on the same context is still correct.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_sets_status_and_context_stays_usable():
    from lookahead_keys_attention_b200 import _lib as L, castle_attention, check_status
    from lookahead_keys_attention_b200.ops import status_word
    from oracle import castle_oracle as O
    lib = L.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    check_status()                       # start from a clean word
    st = status_word(dev)
    polls = torch.full((2,), -1, dtype=torch.int32, device=dev)
    limit = 1024
    L.check(lib.castle_selftest_wait_timeout(limit, polls.data_ptr(), st.data_ptr(), None), "wait_timeout")
    torch.cuda.synchronize()             # the kernel RETURNED: nothing hangs
    n1, n2 = polls.tolist()
    assert 0 <= n1 <= limit              # thread 0 either ran out itself or saw another thread's flag
    assert n2 == 0                       # with the flag up, a later wait gives up at its first poll
    assert int(st.item()) & 1            # CASTLE_STATUS_WAIT_TIMEOUT
    with pytest.raises(RuntimeError, match="bounded wait"):
        check_status()
    assert int(st.item()) == 0           # raising cleared the word
    check_status()

    # the context is intact: an ordinary forward pass is still right
    torch.manual_seed(0)
    t = [(torch.randn(1, 2, 200, 64) * 3 ** -0.5).bfloat16() for _ in range(6)]
    out = castle_attention(*[x.cuda() for x in t], 0.125)
    ref = O.castle_parallel(*[x.float() for x in t], 0.125)
    torch.cuda.synchronize()
    check_status()
    err = (out.float().cpu() - ref).abs()
    assert bool((err <= 2e-2 + 1e-2 * ref.abs()).all()), err.max().item()


def test_wait_timeout_selftest_rejects_bad_arguments():
    from lookahead_keys_attention_b200 import _lib as L
    lib = L.load()
    z = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert lib.castle_selftest_wait_timeout(0, z.data_ptr(), z.data_ptr(), None) < 0
    assert lib.castle_selftest_wait_timeout(1 << 20, z.data_ptr(), z.data_ptr(), None) < 0
    assert lib.castle_selftest_wait_timeout(16, None, z.data_ptr(), None) < 0
