/* TEST INFRASTRUCTURE ONLY -- CPU oracle for the fbw (fast Baum-Welch) path.
 *
 * A plain-C restatement of the arithmetic of the reference's CUDA-only op
 * (i6_native_ops/fbw/fbw_op.cu:226-393; the reference has no CPU implementation of fbw, its
 * binding rejects CPU tensors at i6_native_ops/fbw/fbw_torch.cpp:19-23).  It is the checker for
 * the CUDA kernels and the timed CPU baseline of the benchmark; nothing in the shipped package
 * imports, links or runs it.
 *
 * Two entry points with identical argument lists:
 *   fbw_oracle_f32  -- fp32 arithmetic in the reference's operation order (ascending edge index
 *                      wherever the reference accumulates), expf/log1pf from the host libm.
 *                      Host libm is not bit-identical to CUDA's libdevice, so this mode agrees
 *                      with the GPU reference to a few ulp of the score magnitude, not bitwise.
 *   fbw_oracle_f64  -- the same recursion in double precision ("truth").
 *
 * Parity pin: the reference's own tests hold no loss or posterior values for fbw (test/fbw.py
 * checks only that posteriors sum to one).  The oracle is therefore pinned against outputs of
 * the reference op itself, produced on a GPU by tests/golden/make_golden.py and committed as
 * fixtures, plus brute-force path enumeration and torch's CTC loss.
 *
 * Arguments: am (T,B,F) negative log scores; edges (4,E) rows from/to/emission/sequence;
 * weights (E); start_end (2,B); seq_lens (B); S = number of states (global id space);
 * out (T,B,F) negative log posteriors, +inf where zero; sums (T,B) per-frame normalisers
 * (0 for frames at or past seq_len); alpha_out / beta_out optional ((T+1),S) state scores,
 * may be NULL.  Returns 0, or a small positive code for malformed input.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#define CAT2(a, b) a##b
#define CAT(a, b) CAT2(a, b)

#define REAL float
#define NAME(x) CAT(x, _f32)
#define EXP expf
#define LOG1P log1pf
#define FMIN fminf
#define FABS fabsf
#include "fbw_oracle_impl.inc"
#undef REAL
#undef NAME
#undef EXP
#undef LOG1P
#undef FMIN
#undef FABS

#define REAL double
#define NAME(x) CAT(x, _f64)
#define EXP exp
#define LOG1P log1p
#define FMIN fmin
#define FABS fabs
#include "fbw_oracle_impl.inc"
