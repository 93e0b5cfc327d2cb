"""Developer aid: cycles per tensor-core instruction (128 x n x 16, 16-bit operands from shared memory)
for each operand form and width, measured by `castle_selftest_mma_rate` on one SM.

    python -m lookahead_keys_attention_b200.mma_rate

Each line is the slope between a 64- and a 512-instruction run, so launch and commit latency cancel.
"""
import torch

from . import _lib as L

FORMS = ["A rows, B rows", "A rows, B cols", "A cols, B cols", "A cols, B rows"]


def measure(lib, form, n, reps, cyc, st):
    rc = lib.castle_selftest_mma_rate(form, n, reps, cyc.data_ptr(), st.data_ptr(), None)
    if rc:
        raise RuntimeError(L.last_error())
    torch.cuda.synchronize()
    if int(st.item()):
        raise RuntimeError(f"device status {int(st.item())}")
    issue, total = cyc.cpu().tolist()
    return issue, total


def main():
    lib = L.load()
    cyc = torch.zeros(2, dtype=torch.int64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    print("cycles per 128 x n x 16 product (issue-to-completion slope; operand bytes read from shared memory)")
    for n in (64, 128, 192, 256):
        for form, name in enumerate(FORMS):
            i1, t1 = measure(lib, form, n, 64, cyc, st)
            i2, t2 = measure(lib, form, n, 512, cyc, st)
            per = (t2 - t1) / 448
            smem = 128 * 32 + n * 32
            print(f"  n={n:3d}  {name:15s} {per:6.1f} cycles   {smem / per:6.1f} B/cycle of operands,"
                  f" {128 * n * 16 * 2 / per:7.0f} flop/cycle")


if __name__ == "__main__":
    main()
