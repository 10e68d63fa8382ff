/* fbw_b200.h -- C ABI of the B200 (sm_100a) full-sum forward-backward ("fast Baum-Welch") op.
 *
 * This is the boundary a host binding links against.  Together the calls below replace the
 * reference's host launcher  fbw_cuda()  (i6_native_ops/fbw/fbw_op.cu:226-393), which its
 * binding  fbw()  (i6_native_ops/fbw/fbw_torch.cpp:15-29) calls with the same five arrays.
 *
 * All pointers are DEVICE pointers unless a comment says host.  Sizes are 64-bit.  The score tensor
 * handed to fbw_b200_run / _run_fused / _viterbi may be ANY memory the device can address, in
 * particular pinned host memory under unified addressing: the ops read it exactly once, and only the
 * scores the automata refer to (one 32-byte sector per distinct frame/sequence/emission), so scores
 * produced on the host need not be copied to the device as a whole.  No call
 * allocates device memory; scratch is passed in by the caller.  Calls enqueue work on the given
 * stream and return without synchronising, except fbw_b200_plan_summary.
 *
 * Call order for one op call:
 *     plan  = caller-allocated  fbw_b200_plan_bytes(B, E, S)  bytes
 *     fbw_b200_prepare(...)                      -- validates the automata, builds sorted edge lists
 *     fbw_b200_plan_summary(plan, &sum, stream)  -- host gets sizes + validation result (synchronises)
 *     work  = caller-allocated  fbw_b200_run_bytes(&sum)  bytes
 *     fbw_b200_run(...)                          -- scores -> out, sums (and optional loss scalars)
 * A plan depends only on the automata and seq_lens; it can be kept and reused with new scores.
 */
#ifndef FBW_B200_H
#define FBW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* CUDA stream handle (cudaStream_t / CUstream) without pulling in CUDA headers. */
typedef struct CUstream_st* fbw_b200_stream_t;

/* Status codes (0 = success).  fbw_b200_status_string() gives the text.  The reference reports
 * the same classes of failure as TORCH_CHECK errors / asserts
 * (i6_native_ops/common/returnn_definitions.h:82-123). */
enum {
    FBW_B200_OK             = 0,
    FBW_B200_BAD_ARGUMENT   = 1, /* null pointer, non-positive dimension, misaligned buffer      */
    FBW_B200_WORKSPACE      = 2, /* caller-provided scratch too small                            */
    FBW_B200_CUDA_ERROR     = 3, /* a CUDA runtime call failed (see cudaGetLastError)            */
    FBW_B200_BAD_AUTOMATON  = 4, /* summary.error != 0: an index in edges/start_end out of range,
                                    a state used by two sequences, or a per-sequence size limit */
    FBW_B200_TOO_LARGE      = 5, /* request exceeds the fixed capacity of a no-allocation entry  */
    FBW_B200_RETRY_GENERAL  = 6  /* fbw_b200_prepare took its fast path and a sequence did not fit it:
                                    call fbw_b200_prepare_general with the same arguments        */
};

/* Bits of fbw_b200_summary.error (validation of the automata; the reference does not validate,
 * out-of-range input is undefined behaviour there). */
enum {
    FBW_B200_ERR_STATE_RANGE    = 1,  /* from/to state id outside [0, S)                  */
    FBW_B200_ERR_EMISSION_RANGE = 2,  /* emission id outside [0, F)                       */
    FBW_B200_ERR_SEQ_RANGE      = 4,  /* sequence id outside [0, B)                       */
    FBW_B200_ERR_START_END      = 8,  /* start or end state outside [0, S)                */
    FBW_B200_ERR_SHARED_STATE   = 16, /* one state id used by edges of two sequences      */
    FBW_B200_ERR_SEQ_TOO_LARGE  = 32, /* a sequence has more than 65535 states or classes */
    FBW_B200_ERR_RETRY_GENERAL  = 64  /* not an input error: see FBW_B200_RETRY_GENERAL    */
};

#define FBW_B200_GROUPS 8

/* Sizes the host needs after fbw_b200_prepare (HOST struct). */
typedef struct fbw_b200_summary {
    int64_t error;        /* validation bits above; 0 = automata accepted                         */
    int64_t T, B, F, E, S;
    int64_t state_floats; /* floats in each of the two per-frame state-score arrays (alpha, beta) */
    int64_t tiled_floats; /* floats in the tiled gathered-score array                              */
    int64_t frame_floats; /* floats in each frame-major array (gathered scores, class posteriors) */
    int64_t num_slots;    /* sum over sequences of distinct emission classes                      */
    int64_t max_states, max_edges, max_slots, max_len; /* per-sequence maxima                    */
    int64_t sum_len;      /* sum over sequences of valid frames                                   */
    int64_t gather_units, post_units; /* work items of the gather / posterior kernels             */
    /* Sequences are ranked by cost (frames x edges, descending); group g is the rank range
     * [g*B/FBW_B200_GROUPS, (g+1)*B/FBW_B200_GROUPS).  Per-group maxima size each group's launch. */
    int64_t group_max_states[8], group_max_edges[8], group_max_slots[8];
    int64_t max_degree;   /* largest in-degree or out-degree of a state                           */
    int64_t score_floats; /* floats in the per-frame edge-score array                              */
    int64_t min_len;      /* shortest valid sequence length (0 if none)                           */
    int64_t reserved[1];
} fbw_b200_summary;

/* Bytes of plan scratch for B sequences, E edges, S states. */
size_t fbw_b200_plan_bytes(int64_t B, int64_t E, int64_t S);

/* Validate the automata and build the per-sequence sorted edge lists into `plan`.
 * edges (4,E) int32 rows from/to/emission/sequence, weights (E) f32, start_end (2,B) int32,
 * seq_lens (B) int32 -- the layouts of fbw_op.cu:249-263.  T,B,F are the dims of the score tensor.
 * Replaces nothing in the reference one-to-one: the reference walks the unsorted edge list with
 * atomics every frame (next_frame, fbw_op.cu:71-102); sorting once removes the atomics. */
int fbw_b200_prepare(const int32_t* edges, const float* weights, const int32_t* start_end,
                     const int32_t* seq_lens, int64_t T, int64_t B, int64_t F, int64_t E, int64_t S,
                     void* plan, size_t plan_bytes, fbw_b200_stream_t stream);

/* The same, always through the general path (device-wide radix sorts; any sequence size within the
 * limits above).  fbw_b200_prepare itself picks a faster path (one CTA sorts one sequence in shared
 * memory) when the average sequence is small; if a single sequence then exceeds that path's capacity
 * (4096 edges), fbw_b200_plan_summary returns FBW_B200_RETRY_GENERAL and this call redoes the plan. */
int fbw_b200_prepare_general(const int32_t* edges, const float* weights, const int32_t* start_end,
                             const int32_t* seq_lens, int64_t T, int64_t B, int64_t F, int64_t E,
                             int64_t S, void* plan, size_t plan_bytes, fbw_b200_stream_t stream);

/* Copy the plan's summary to host memory.  SYNCHRONISES the stream.  Returns
 * FBW_B200_BAD_AUTOMATON if validation failed (summary->error says why), FBW_B200_RETRY_GENERAL if
 * the plan has to be redone with fbw_b200_prepare_general. */
int fbw_b200_plan_summary(const void* plan, fbw_b200_summary* summary, fbw_b200_stream_t stream);

/* Bytes of run scratch for a prepared plan. */
size_t fbw_b200_run_bytes(const fbw_b200_summary* summary);

/* The op: am (T,B,F) f32 negative log scores -> out (T,B,F) f32 negative log class posteriors
 * (+inf where zero and for frames t >= seq_len) and sums (T,B) f32 per-frame normalisers
 * (0 for t >= seq_len or when no path exists): the two tensors fbw_cuda returns
 * (fbw_op.cu:230-232, 392).  Covers the alpha/beta initialisation (fbw_op.cu:297-302, 61-69),
 * both sweeps (318-353), the normaliser (104-135) and the scatter into the output (137-153,
 * 366-378).  loss2 (2 floats, may be NULL): [0] = sum of all sums, [1] = sum over sequences of
 * sums[0,b]; written by the last kernel so a collective can follow on the same stream. */
int fbw_b200_run(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                 float* sums, float* loss2, void* work, size_t work_bytes,
                 fbw_b200_stream_t stream);

/* fbw_b200_run for a call whose forward state scores will be exported (fbw_b200_export_alpha): same
 * arguments, same `out` and `sums` bit for bit.  The plain run leaves at +inf the scores of states
 * that cannot lie on a complete path (too few frames left to reach the end state), which no output
 * depends on; this variant computes them as the reference does (fbw_op.cu:71-102 relaxes every edge),
 * so that the exported forward scores equal the reference's state buffer (fbw_op.cu:304-315). */
int fbw_b200_run_for_export(const void* plan, const fbw_b200_summary* summary, const float* am,
                            float* out, float* sums, float* loss2, void* work, size_t work_bytes,
                            fbw_b200_stream_t stream);

/* fbw_b200_run for callers whose results live in host memory: same arguments, plus `out_host`, a
 * PINNED HOST buffer of T*B*F floats that receives a copy of `out` (which stays a device buffer).  The
 * copy is part of the call: large calls that run as a pipeline over time chunks send every finished
 * part of the (T,B,F) output to the host (cudaMemcpyAsync on a library-owned stream) while the rest is
 * still being computed, so the device -> host transfer, which takes longer than the op, starts early;
 * other calls copy once at the end.  The copy is joined into `stream` before the call returns (the
 * call still only enqueues).  No counterpart in the reference, whose outputs are device tensors. */
int fbw_b200_run_host_out(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                          float* out_host, float* sums, float* loss2, void* work, size_t work_bytes,
                          fbw_b200_stream_t stream);

/* fbw_b200_run for callers whose scores and/or results live in PINNED HOST memory, with host threads of
 * this library (as many as the process may use, at most 16; FBW_B200_HOST_THREADS) taking over what is
 * slow over the bus.  Arguments as fbw_b200_run; `am` and `out` may each be device memory or pinned host
 * memory (device-accessible under unified addressing); `host_work`: PINNED HOST scratch, 256-byte
 * aligned, of fbw_b200_run_with_host_bytes(summary) bytes, the caller's as all scratch is.
 *   Scores in host memory: the device would fetch the entries the automata refer to as 32-byte reads
 * over the bus, and nothing else of the call can start before.  The host threads pick them out of the
 * tensor instead and one copy takes them to the device (triphone workload: 14 ms against 37 ms).
 *   Result in host memory, sparse rows (few classes per sequence against F): sending the (T,B,F) result
 * over the bus would cost more than computing it, and nearly all of it is +inf.  The device sends only
 * the class posteriors (2 % of the result on the triphone workload), into `host_work`, as its posterior
 * stages finish, and the host threads write the rows from them while the device goes on.  Dense rows
 * are written whole by the device's output pass, straight into `out`.
 * THE CALL BLOCKS while the host threads work: with scores in host memory before the device work is
 * enqueued, with host-written rows until they are written, so that a host `out` is complete when the
 * call returns; `sums`, `loss2` and a device `out` are complete when `stream` has been synchronised, as
 * for every other entry.  One such call per device at a time (others wait).  Same bits as fbw_b200_run.
 * No counterpart in the reference, whose inputs and outputs are device tensors. */
size_t fbw_b200_run_with_host_bytes(const fbw_b200_summary* summary);
int fbw_b200_run_with_host(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                           float* sums, float* loss2, void* work, size_t work_bytes, void* host_work,
                           size_t host_work_bytes, fbw_b200_stream_t stream);

/* fbw_b200_run with the Python wrapper's elementwise passes folded in (the steps either side of the
 * op in i6_native_ops/fbw/__init__.py:41-44 and :66): the input is log_probs in the caller's own
 * (B,T,F) layout and sign (prepare was given T, B, F of that tensor), the output `grad` (B,T,F) is
 * d(sum of sums)/d(log_probs) = -posterior, 0 where the posterior is 0 and for t >= seq_len.  `sums`
 * (T,B) and loss2 as in fbw_b200_run.  Saves four passes over the (B,T,F) tensor per training step. */
int fbw_b200_run_fused(const void* plan, const fbw_b200_summary* summary, const float* log_probs,
                       float* grad, float* sums, float* loss2, void* work, size_t work_bytes,
                       fbw_b200_stream_t stream);

/* Best-path (Viterbi) alignment on the same plan: replaces the reference's second FSA op,
 * fast_viterbi_cuda()  (i6_native_ops/fast_viterbi/core.cu:174-275), which its binding
 * fast_viterbi()  (i6_native_ops/fast_viterbi/binding.cpp:13-25) calls with the same five arrays.
 * `scores_in` holds POSITIVE log scores (larger is better), (T,B,F) f32.  Outputs, as core.cu:274:
 * `alignment` (T,B) i32 = emission id of the best path's edge at each frame, 0 for frames
 * t >= seq_len and where no edge was recorded; `scores` (B) f32 = value of the best path ending
 * in the end state after seq_len frames (-inf if there is none).  Ties are broken as in the
 * reference (core.cu:37-40): the smaller edge index wins, so alignment and scores are reproduced
 * bit for bit.  A seq_len outside [0, T] (the reference then reads past its table) is treated as 0.
 * batch_major != 0 folds in the wrapper's two transposes (i6_native_ops/fast_viterbi/__init__.py:37,
 * 46): `scores_in` is the caller's (B,T,F) log_probs and `alignment` is written as (B,T).
 * The plan is the one fbw_b200_prepare builds (same automata, same seq_lens); `work` needs
 * fbw_b200_viterbi_bytes(summary) bytes, 256-byte aligned.  Enqueues on `stream`, no synchronisation. */
size_t fbw_b200_viterbi_bytes(const fbw_b200_summary* summary);
int fbw_b200_viterbi(const void* plan, const fbw_b200_summary* summary, const float* scores_in,
                     int32_t* alignment, float* scores, int batch_major, void* work,
                     size_t work_bytes, fbw_b200_stream_t stream);

/* fbw_b200_viterbi for scores in PINNED HOST memory, with the library's host threads picking the entries
 * the automata refer to out of the tensor (see fbw_b200_run_with_host, whose scratch size
 * fbw_b200_run_with_host_bytes also holds here).  The call blocks while they work, before the device work
 * is enqueued.  Scores in device memory are accepted and handled as by fbw_b200_viterbi.  Same results. */
int fbw_b200_viterbi_with_host(const void* plan, const fbw_b200_summary* summary, const float* scores_in,
                               int32_t* alignment, float* scores, int batch_major, void* work,
                               size_t work_bytes, void* host_work, size_t host_work_bytes,
                               fbw_b200_stream_t stream);

/* fbw_b200_run with per-phase device timing, for benchmarks and profiles: same arguments and
 * results, plus phase_ms (HOST, FBW_B200_NUM_PHASES floats) = milliseconds of the gather, sweep,
 * posterior, expand and loss-reduction kernels measured with CUDA events on `stream`.
 * SYNCHRONISES the stream and creates/destroys events; not for production use.  No counterpart in
 * the reference (it has no timing code in fbw). */
#define FBW_B200_NUM_PHASES 5
int fbw_b200_run_phases(const void* plan, const fbw_b200_summary* summary, const float* am,
                        float* out, float* sums, float* loss2, void* work, size_t work_bytes,
                        fbw_b200_stream_t stream, float* phase_ms);

/* Debug export for the text dumps of the reference (write_alignment_to_file, fbw_op.cu:155-195, which
 * reads the per-frame forward state buffer kept at fbw_op.cu:304-315, 327-331): copies the forward
 * state scores alpha_t(s) that the LAST fbw_b200_run / fbw_b200_run_fused left in `work` into `alpha`,
 * a dense (T, S) f32 array indexed by frame and GLOBAL state id.  +inf for unreachable states, for
 * state ids no sequence uses and for frames t >= seq_len; row 0 of a sequence without valid frames is
 * its initial vector (0 at the start state).  Enqueues on `stream`; `work` must not have been reused. */
int fbw_b200_export_alpha(const void* plan, const fbw_b200_summary* summary, const void* work,
                          size_t work_bytes, float* alpha, fbw_b200_stream_t stream);

/* Device-side builders of the automaton tensors (edges (4,E) i32, weights (E) f32, start_end (2,B)
 * i32, num_states) from label sequences.  No counterpart in the reference, whose automata come from an
 * external exporter (only the tuple format is defined, i6_native_ops/fbw/__init__.py:49-63).
 * Two steps, because the edge count depends on the labels:
 *   *_count  writes per-sequence offsets into `scratch` (fbw_b200_topology_bytes(B) bytes, 256-byte
 *            aligned) and returns the totals in HOST variables (SYNCHRONISES the stream);
 *   *_fill   writes the tensors the caller allocated with those totals (enqueue only).
 * State ids are global and consecutive per sequence.
 * CTC: labels (B,Lmax) i32, label_lens (B) i32.  Local states 0..2L alternate blank/label plus one
 *   separate final state 2L+1; an edge emits its target's symbol; loop, advance, and skip between
 *   different labels; each edge entering one of the last two states has a copy entering the final
 *   state; weights 0; start = first state, end = final state.
 * HMM chain: classes (B,Nmax) i32, lens (B) i32, optional (B,Nmax) u8 or NULL.  Virtual start state 0,
 *   state i+1 carries classes[i]; edge 0->1 weight 0; per state a loop (loop_weight), a forward edge
 *   (forward_weight) and a j->j+2 edge: everywhere with skip_weight if skip_all != 0, else with
 *   forward_weight around the states whose `optional` flag is set.  Weights are negative log values. */
size_t fbw_b200_topology_bytes(int64_t B);
int fbw_b200_ctc_topology_count(const int32_t* labels, const int32_t* label_lens, int64_t B,
                                int64_t Lmax, int32_t blank, void* scratch, size_t scratch_bytes,
                                int64_t* num_states, int64_t* num_edges, fbw_b200_stream_t stream);
int fbw_b200_ctc_topology_fill(const int32_t* labels, const int32_t* label_lens, int64_t B,
                               int64_t Lmax, int32_t blank, const void* scratch, int64_t num_edges,
                               int32_t* edges, float* weights, int32_t* start_end,
                               fbw_b200_stream_t stream);
int fbw_b200_hmm_topology_count(const int32_t* lens, const uint8_t* optional, int64_t B, int64_t Nmax,
                                int skip_all, void* scratch, size_t scratch_bytes,
                                int64_t* num_states, int64_t* num_edges, fbw_b200_stream_t stream);
int fbw_b200_hmm_topology_fill(const int32_t* classes, const int32_t* lens, const uint8_t* optional,
                               int64_t B, int64_t Nmax, float loop_weight, float forward_weight,
                               float skip_weight, int skip_all, const void* scratch,
                               int64_t num_edges, int32_t* edges, float* weights, int32_t* start_end,
                               fbw_b200_stream_t stream);

/* Number of kernels of this library launched by this process so far (its own kernels only, not
 * the CUB sort/scan kernels it calls during prepare).  No counterpart in the reference. */
int64_t fbw_b200_launch_count(void);

/* The whole op (prepare + summary + run) for callers that cannot allocate device memory while they
 * run -- for example a server whose memory pool is fixed at start-up, or a plug-in that only ever
 * receives input and output buffers from its host and has no allocator to ask for scratch.  The plan
 * and the run scratch live in a fixed array inside the library (fbw_b200_noalloc_capacity() bytes,
 * 64 MiB, held by every GPU that loads the library until the process exits).  Same inputs and
 * outputs as fbw_b200_prepare + fbw_b200_run; loss2 may be NULL.  It has no counterpart in the
 * reference, whose launcher allocates and frees per call (fbw_op.cu:283-286, 384-389).
 *  - Returns FBW_B200_TOO_LARGE when plan + scratch exceed the capacity, or when T*B*F >= 1e8 (a fixed
 *    cap: this entry runs its stages one after another on the caller's stream, which suits small and
 *    medium calls).  `out`, `sums` and `loss2` are untouched then; if only the run scratch did not fit,
 *    the plan kernels have already run on the array and the stream has been synchronised.
 *  - Calls no cudaMalloc/cudaFree and no allocating library routine.  SYNCHRONISES the stream on
 *    every call (the host reads the plan summary), so it cannot be part of a stream capture.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, that
 *    device current); make that first call before any stream capture starts on that device.
 *  - All calls on a device share the one array: two calls that overlap on the GPU (different
 *    streams or threads) race on it.  The array keeps the previous call's contents; everything a call
 *    needs to start from zero it clears itself. */
int fbw_b200_fbw_noalloc(const float* am, const int32_t* edges, const float* weights,
                         const int32_t* start_end, const int32_t* seq_lens, int64_t T, int64_t B,
                         int64_t F, int64_t E, int64_t S, float* out, float* sums, float* loss2,
                         fbw_b200_stream_t stream);
size_t fbw_b200_noalloc_capacity(void);

/* Text for a status code (static storage). */
const char* fbw_b200_status_string(int status);

/* ABI version of this header. */
int fbw_b200_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FBW_B200_H */
