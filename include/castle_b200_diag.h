/* castle_b200_diag.h - diagnostics of the B200 CASTLE attention library.
 *
 * NOT part of the drop-in ABI (include/castle_b200.h): nothing here has a
 * counterpart in the reference, and a host that only runs attention never
 * needs it.  These entry points exist for the repository's own tests and
 * benchmark: a self test of the tensor-core operand forms the kernels rely
 * on, an instruction-rate probe, a test of the bounded-wait failure path, and
 * CUDA-event hooks around the main kernels.  Same conventions as the ABI
 * header (return codes, caller-owned buffers, asynchronous launches).
 */
#ifndef CASTLE_B200_DIAG_H
#define CASTLE_B200_DIAG_H

#include "castle_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- measurement aid ------------------------------------------------------
 * (no counterpart in the reference)  Bracket the MAIN kernel of later calls (from
 * any host thread of the process) with two caller-owned CUDA events recorded on the launch
 * stream: which = 0 forward, 1 backward, 2 decode step.  Pass NULL events to
 * stop.  Lets a benchmark time the dominant kernel alone, without a profiler.
 */
enum { CASTLE_KERNEL_FWD = 0, CASTLE_KERNEL_BWD = 1, CASTLE_KERNEL_DECODE = 2 };
int castle_set_kernel_events(int32_t which, void* start_event, void* stop_event);

/* ---- self test -------------------------------------------------------------
 * Runs one 128x128 tensor-core product through each operand form the kernels
 * use (no counterpart in the reference).  `x`, `y`: bf16 [128][128] device
 * buffers; `d`: fp32 [128][128].  mode 0: d = x @ y^T; 1: d = x @ y;
 * 2: d = x^T @ y; 3: d = x^T @ y^T; 4: d = 1 - x @ y^T (preset accumulator,
 * negated operand); 5..8: as 0..3 with operands staged by TMA instead of
 * thread stores; 9: d = x @ y^T and 10: d = x @ y with x read from tensor
 * memory (packed 16-bit pairs) instead of shared memory.
 */
int castle_selftest_mma(int32_t mode, const void* x, const void* y, float* d, int32_t* status, void* stream);

/* Measurement aid (no counterpart in the reference): `reps` back-to-back 128 x n x 16 tensor-core
 * products in one operand form (0: both operands read along rows, 1: B read down its columns,
 * 2: both read down their columns, 3: A read down its columns), n in {64, 128, 192, 256}.
 * cycles[0] = SM cycles spent issuing, cycles[1] = cycles from first issue to completion
 * (device pointer to two int64). */
int castle_selftest_mma_rate(int32_t form, int32_t n, int32_t reps, long long* cycles, int32_t* status, void* stream);

/* Failure-path test (no counterpart in the reference): one CTA waits on an mbarrier that nothing
 * ever arrives on, with a poll limit of `poll_limit` (1 .. 65536) instead of the kernels' 2^22.
 * The wait gives up, raises the CTA's abort flag, the kernel falls through a second wait (which
 * must return at once), frees its tensor memory and ORs CASTLE_STATUS_WAIT_TIMEOUT into `status`:
 * the same path every production kernel takes when a wait runs out.  Nothing hangs or faults.
 * polls[0] receives the number of polls the first wait made, polls[1] the second (device int32[2]). */
int castle_selftest_wait_timeout(int32_t poll_limit, int32_t* polls, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CASTLE_B200_DIAG_H */
