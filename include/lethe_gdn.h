/* C interface of liblethe_gdn.so: the chunked gated-delta-rule (GDN family) forward and backward on
 * NVIDIA B200 (sm_100a).
 *
 * It replaces, behind one pair of calls, what the reference project (RishiShah99/lethe) spreads over
 * its autograd op and its kernel plug-ins:
 *   - forward:  src/lethe/kernels/ops/gdn_layer.py:17-67 (_GDN2Function.forward, which today runs the
 *               token-serial src/lethe/kernels/references/gdn_backward.py:13-55 or the chunkwise
 *               restage src/lethe/kernels/references/gdn2_chunkwise_cw.py:213-314);
 *   - backward: src/lethe/kernels/ops/gdn_backward.py:16-57 -> src/lethe/kernels/cute/gdn2_backward.py:77-134
 *               -> src/lethe/kernels/cute/gdn2_assemble.py:242-314 / :601-696 / :711-775, i.e. the
 *               forward recompute, the reverse state scan K#1 (K1Fn, gdn2_assemble.py:29-32), the
 *               closed Stage B (:521-585) and the WY / triangular-inverse VJP K#2 (K2Fn, :33-44).
 *
 * Ownership: the caller allocates every buffer (inputs, outputs, the two workspaces and the status
 * word) on one GPU; the library works on the GPU that owns `q` (it need not be the calling thread's
 * current device), allocates nothing and keeps no state between calls.
 * Threading: re-entrant; all work is enqueued on the given stream; no call synchronises.
 * Errors: a non-zero return means nothing was launched (see lethe_gdn_strerror).  Device-side waits
 * are bounded; a wait that gave up leaves a non-zero code in *status, readable once the stream has
 * been synchronised (results are then invalid).  The caller zeroes *status before the first call.
 *
 * Layouts (all row-major, innermost dimension contiguous):
 *   q, k        [B, L, H, K]  bf16          v, o, do, dv [B, L, H, V]  bf16     dq, dk [B, L, H, K] bf16
 *               (q, k, dq, dk: fp16 when args->qk_f16 is set)
 *   g           [B, L, H] (gate = 1) or [B, L, H, K] (gate = 2), fp32, natural-log decay (<= 0)
 *   beta        [B, L, H] fp32 (delta = 1)
 *   h0, hT, dhT, dh0   [B, H, K, V] fp32
 *   dg          like g, fp32;   dbeta like beta, fp32
 * Sizes: K = 128, V in {64, 128}, L a multiple of 64 (the chunk length).
 */
#ifndef LETHE_GDN_H_
#define LETHE_GDN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { LETHE_GATE_NONE = 0, LETHE_GATE_SCALAR = 1, LETHE_GATE_CHANNEL = 2 };

typedef struct LetheGdnDims {
  int32_t B, H, L, K, V;
  int32_t gate;   /* LETHE_GATE_*                                                        */
  int32_t delta;  /* 1: erase and write gates are beta (gated delta rule, KDA)            */
                  /* 0: no erase term, write gate one (linear attention, GLA, SSD)        */
                  /* 2: independent per-channel erase gate b and write gate w, the full   */
                  /*    op of the reference (gdn_backward.py:45-53); needs the            */
                  /*    channel-wise gate                                                 */
} LetheGdnDims;

typedef struct LetheGdnArgs {
  LetheGdnDims dims;
  float scale;            /* multiplies q; the reference default is K^-0.5                  */
  /* forward inputs */
  const void* q;
  const void* k;
  const void* v;
  const float* g;         /* NULL when gate == LETHE_GATE_NONE                              */
  const float* beta;      /* NULL when delta == 0                                           */
  const float* h0;        /* NULL: zero initial state                                       */
  /* forward outputs */
  void* o;
  float* hT;              /* NULL: final state not wanted                                   */
  /* backward inputs */
  const void* d_o;
  const float* dhT;       /* NULL: zero                                                     */
  /* backward outputs */
  void* dq;
  void* dk;
  void* dv;
  float* dg;              /* NULL when gate == LETHE_GATE_NONE                              */
  float* dbeta;           /* NULL when delta == 0                                           */
  float* dh0;             /* NULL: not wanted                                               */
  /* caller-owned scratch */
  void* saved;            /* written by forward, read by backward; lethe_gdn_saved_bytes     */
  size_t saved_bytes;
  void* scratch;          /* backward only; lethe_gdn_scratch_bytes                          */
  size_t scratch_bytes;
  int32_t* status;        /* device word, see above                                         */
  /* Profiling aid: 0 runs every kernel of the call.  Otherwise bit i selects kernel i of the call  */
  /* (forward: 1 prepare, 2 state scan, 4 output; backward: 1 scan input, 2 adjoint scan,           */
  /* 4 Stage B, 8 WY VJP); a partial call relies on the records left by an earlier full call.       */
  uint32_t kernel_mask;
  /* Optional split of the beta gradient (delta = 1).  NULL: `dbeta` receives the whole gradient.     */
  /* Non-NULL: `dbeta` receives the erase-gate part and `dbeta_write` the write-gate part, the two    */
  /* gradients the reference returns separately (db_erase / dw_write, gdn2_assemble.py:150-181).      */
  float* dbeta_write;
  /* delta = 2 only (NULL otherwise): erase gate b [B, L, H, K] and write gate w [B, L, H, V], fp32,     */
  /* and their gradients (backward).  `beta` / `dbeta` are not used in this mode.                       */
  const float* b_gate;
  const float* w_gate;
  float* db_gate;
  float* dw_gate;
  /* The (batch, head) pairs this call works on: pairs [bh_begin, bh_begin + bh_count) in b * H + h order;     */
  /* bh_count = 0 means all of them.  Pairs are independent recurrences: calls on disjoint ranges may run     */
  /* concurrently on different streams with the same tensors and workspaces (no counterpart in the reference). */
  uint32_t bh_begin;
  uint32_t bh_count;
  /* Non-zero: q, k (inputs) and dq, dk (outputs) hold IEEE fp16 instead of bf16.  fp16 is the type of the  */
  /* tensor-core operands, so a caller that forms q, k in fp32 (the L2 normalisation below) rounds them      */
  /* once, as the reference does when it stages operands (gdn2_bwd_dhu_l3.py:477-479), instead of twice.     */
  /* v, o, d_o, dv stay bf16.                                                                               */
  uint32_t qk_f16;
  /* The chunks (64-token blocks) of every sequence this call works on: [c_begin, c_begin + c_count); c_count = 0  */
  /* means all L / 64 of them.  The chunk-parallel kernels simply cover that range.  The state scans carry    */
  /* their fp32 state from one range to the next through the workspaces, so the forward ranges must be run    */
  /* in ascending order and the backward ranges in descending order (kernel_mask selects the kernels): a      */
  /* call cut into ranges gives bit-identical results and lets a caller overlap the chunk-parallel kernels    */
  /* of one range with the serial scan of the next on another stream (lethe_b200.ops.GdnStepGraph does).      */
  /* No counterpart in the reference.                                                                          */
  uint32_t c_begin;
  uint32_t c_count;
} LetheGdnArgs;

/* Bytes of the forward->backward workspace / of the backward scratch for these sizes (0 = bad dims). */
size_t lethe_gdn_saved_bytes(const LetheGdnDims* dims);
size_t lethe_gdn_scratch_bytes(const LetheGdnDims* dims);

/* Forward: o (and hT) from q, k, v, g, beta, h0.  Replaces gdn_layer.py:17-67 of the reference. */
int lethe_gdn_forward(const LetheGdnArgs* args, void* cuda_stream);

/* Backward: dq, dk, dv, dg, dbeta, dh0 from the forward inputs, d_o, dhT and `saved`.
 * Replaces gdn_backward.py:16-57 / gdn2_assemble.py:242-314,601-696,711-775 of the reference. */
int lethe_gdn_backward(const LetheGdnArgs* args, void* cuda_stream);

/* Forward without a caller-supplied workspace, for hosts that cannot allocate device memory (a
 * plug-in inside a runtime whose memory pool is off limits, a server that fixed its memory budget
 * at start-up).  It has no counterpart in the reference.  Same arguments and results as
 * lethe_gdn_forward, except that args->saved / saved_bytes are ignored: the per-chunk records go
 * through a 16 MiB array built into the library (lethe_gdn_forward_static_capacity()), so
 *   - the problem must satisfy lethe_gdn_saved_bytes(dims) <= 16 MiB, else the call returns the
 *     "needs more workspace" error and launches nothing;
 *   - the records are not kept for a backward pass (inference / evaluation only);
 *   - all calls on one GPU share the array: calls that could overlap on the GPU must be put on one
 *     stream; nothing needs clearing between calls;
 *   - every GPU has its own copy of the array.  The call works on the GPU that owns args->q,
 *     whatever device the calling thread has selected, and uses that GPU's copy;
 *   - the first call for each GPU looks up the array's device address there and may make the driver
 *     load the library's code onto that GPU (this is when the 16 MiB get reserved); make that call
 *     before any stream capture starts.
 * After that first call on a GPU, a call allocates nothing (no cudaMalloc, no cudaFree, no library
 * that would). */
int lethe_gdn_forward_static(const LetheGdnArgs* args, void* cuda_stream);
size_t lethe_gdn_forward_static_capacity(void);

/* One token of the same recurrence for generation (the body of the reference's token loop,
 * src/lethe/kernels/references/gdn_backward.py:45-53; the reference has no device kernel for it):
 *   S <- S * exp(g);  v_new = beta (v - k^T S);  S <- S + k v_new^T;  o = (scale q)^T S
 * for every (batch, head) pair.  q, k: bf16 [B, H, K]; v, o: bf16 [B, H, V]; g: fp32 [B, H] (scalar
 * gate) or [B, H, K] (channel-wise), unused for LETHE_GATE_NONE; beta: fp32 [B, H], required when
 * delta != 0; state: fp32 [B, H, K, V], updated in place (the h_T of lethe_gdn_forward continues a
 * prompt).  K = 128, V in {64, 128}.  No workspace, no status word (the kernel waits on nothing). */
typedef struct LetheGdnDecodeArgs {
  int32_t B, H, K, V;
  int32_t gate;   /* LETHE_GATE_* */
  int32_t delta;  /* 0: no delta term (v_new = v) */
  float scale;
  const void* q;
  const void* k;
  const void* v;
  const float* g;
  const float* beta;
  float* state;
  void* o;
} LetheGdnDecodeArgs;
int lethe_gdn_decode_step(const LetheGdnDecodeArgs* args, void* cuda_stream);

/* L2 normalisation of q and k before the recurrence, and its vector-Jacobian product after the
 * backward (reference src/lethe/kernels/references/gdn_backward.py:9-10, applied at :29-31 when
 * use_qk_l2norm is set; the reference differentiates it by autograd,
 * src/lethe/kernels/references/gdn2_assemble.py:300-312):
 *   y = x * rsqrt(sum_d x_d^2 + eps);      dx = r (dy - y (y . dy)),  r = rsqrt(sum_d x_d^2 + eps).
 * flags: LETHE_L2_IN_F32  - q, k (and the returned dq, dk) are fp32 instead of bf16;
 *        LETHE_L2_NORM_F16 - the normalised rows qn, kn and their gradients dqn, dkn are fp16 instead
 *                            of bf16 (pair it with LetheGdnArgs::qk_f16 on the forward / backward
 *                            calls: the rows are then rounded once, to the operand type).
 * q, k: [rows, D] contiguous; D in {64, 128}; rows = B L H.
 * qn, kn: 16-bit [rows, D], the tensors lethe_gdn_forward / lethe_gdn_backward then read.
 * dqn, dkn: 16-bit [rows, D], the dq / dk lethe_gdn_backward wrote; dq, dk: [rows, D] in the type of
 * q, k (may alias dqn, dkn when both are bf16).  One launch each; every pointer 16-byte aligned. */
enum { LETHE_L2_IN_F32 = 1, LETHE_L2_NORM_F16 = 2 };
int lethe_gdn_l2norm_qk(const void* q, const void* k, void* qn, void* kn, int64_t rows, int32_t D,
                        int32_t flags, float eps, void* cuda_stream);
int lethe_gdn_l2norm_qk_vjp(const void* q, const void* k, const void* dqn, const void* dkn, void* dq, void* dk,
                            int64_t rows, int32_t D, int32_t flags, float eps, void* cuda_stream);

/* Text for a return code of the calls above or for a device status code. */
const char* lethe_gdn_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* LETHE_GDN_H_ */
