// fbw_b200.cu -- full-sum forward-backward (fast Baum-Welch) for B200 (sm_100a).
//
// Replaces the reference's host launcher and kernels (i6_native_ops/fbw/fbw_op.cu:17-153, 226-393)
// behind the C ABI declared in include/fbw_b200.h.  Nothing here is a translation of that file:
// the reference relaxes an unsorted global edge list once per frame with float atomicCAS loops
// (5T+7 launches); this file sorts the automata once per call and then runs five kernels:
//
//   prepare   : validate, number states per sequence, sort edges by target state (forward list),
//               by source state (backward list), by (sequence, emission) and by sequence; rank the
//               sequences by cost.
//   k_gather  : am_scores[t,b,emission] for the distinct emissions of each sequence -> compact
//               score arrays (frame-major for the sweeps, 32-frame tiles for the score pass).
//   k_sweep   : one persistent CTA per (sequence, direction); the automaton lives in shared memory
//               and registers, frames are stepped with one barrier each, next frames' scores arrive
//               by cp.async; state scores leave as full 128-byte lines of a tiled layout.
//   k_score   : time-parallel; edge scores of every (frame, edge), lane = frame.
//   k_norm    : per (sequence, 32 frames): the frame normaliser, a serial left fold.
//   k_class   : per (sequence, 32 frames): the class posteriors.
//   k_expand  : streams the (T,B,F) output: +inf rows with the few finite posteriors patched in.
//   k_patch   : large calls with sparse rows write the output in two steps instead: a warp more per
//               sweep CTA writes the +inf background through the copy engine while the sweeps run
//               (background_rows), and k_patch puts the posteriors into it as whole 32-byte sectors.
// For scores and results in pinned host memory the library's host threads (host_fill.cpp) pick the
// scores out of the tensor and write the result's rows from the posteriors the device sends.
//
// Arithmetic is kept in the reference's fp32 operation order wherever that order is deterministic
// there, because scores grow with t (~2e4 at T=1500, one ulp = 2e-3) and any reassociation shows
// up in the posteriors:
//   * prob_add is fbw_op.cu:39-48 verbatim in meaning: -log1pf(expf(-|a-b|)) + fminf(a,b), +inf for
//     a NaN difference; accurate libdevice expf/log1pf (no fast-math).
//   * an edge's forward value is (alpha + weight) + score (fbw_op.cu:93); the edge score adds beta
//     last (fbw_op.cu:96,99).
//   * the normaliser is a left fold over the sequence's edges in ascending edge index
//     (fbw_op.cu:115-118); state and class accumulations also run in ascending edge index (the
//     reference's atomics have no defined order; with at most two terms the order is immaterial).

#include "fbw_b200.h"
#include "host_fill.h"

#include <cuda_runtime.h>
#include <math_constants.h>

#include <cub/cub.cuh>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace {

constexpr int kTile        = 32;   // frames per tile of the tiled layouts (= one lane per frame)
constexpr int kGatherSlots = 256;  // classes per gather work item
constexpr int kSegFloats   = 512;  // floats per output segment composed in shared memory
constexpr int kMaxPerSeq   = 65535;

typedef long long i64;

// ---------------------------------------------------------------------------------------------
// plan layout (device scratch owned by the caller)
// ---------------------------------------------------------------------------------------------
struct PlanLayout {
    size_t header;
    size_t state_key, skey, skey_out, siota, sorted_state, packed_of;            // [S]
    size_t scount, ecount, unordered, state_off, edge_off, slot_off;             // int[B+1]; unordered: int[4]
    size_t seq_T, start_l, end_l, nslot;                                         // int[B]
    size_t ta_off, tg_off, gf_off, gu_off, pu_off;                               // i64[B+1]
    size_t order, cost;                                                          // int[B], i64[B]
    size_t tx_off;                                                               // i64[B+1]
    size_t qpos, m_pos;                                                          // int[E], int2[E]
    size_t eiota, keyq, keyf, keyb, key32_out, qe, fe, be, me, slot_of_edge;     // [E]
    size_t key64, key64_out;                                                     // u64[E]
    size_t head, hs, m_ptr;                                                      // int[E+1]
    size_t rowcnt_f, rowptr_f, rowcnt_b, rowptr_b;                               // int[S+1]
    size_t fwd_rec, bwd_rec;                                                     // uint2[E]
    size_t q_rec;                                                                // int4[E]
    size_t slot_emis;                                                            // int[E]
    size_t cub_temp, cub_temp_bytes;
    size_t total;
};

size_t cub_temp_need(i64 E, i64 S) {
    // the answer depends on (E, S) only; one call asks three times per op call, so remember the last
    static std::mutex mu;
    static i64 last_E = -1, last_S = -1;
    static size_t last_need = 0;
    std::lock_guard<std::mutex> lk(mu);
    if (E == last_E && S == last_S) return last_need;
    size_t need = 0, b = 0;
    int    nE = (int)(E > 0 ? E : 1), nS = (int)(S > 0 ? S : 1);
    cub::DeviceRadixSort::SortPairs(nullptr, b, (const unsigned*)nullptr, (unsigned*)nullptr,
                                    (const int*)nullptr, (int*)nullptr, nE > nS ? nE : nS);
    need = b > need ? b : need;
    cub::DeviceRadixSort::SortPairs(nullptr, b, (const unsigned long long*)nullptr,
                                    (unsigned long long*)nullptr, (const int*)nullptr,
                                    (int*)nullptr, nE);
    need = b > need ? b : need;
    cub::DeviceScan::ExclusiveSum(nullptr, b, (const int*)nullptr, (int*)nullptr,
                                  (nE > nS ? nE : nS) + 1);
    need = b > need ? b : need;
    last_E = E; last_S = S; last_need = need;
    return need;
}

PlanLayout plan_layout(i64 B, i64 E, i64 S) {
    PlanLayout L;
    size_t     off  = 0;
    auto       take = [&](size_t bytes) {
        size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    size_t nE = (size_t)(E > 0 ? E : 1), nS = (size_t)S, nB = (size_t)B;
    L.header       = take(sizeof(fbw_b200_summary));
    L.state_key    = take(4 * nS);
    L.skey         = take(4 * nS);
    L.skey_out     = take(4 * nS);
    L.siota        = take(4 * nS);
    L.sorted_state = take(4 * nS);
    L.packed_of    = take(4 * nS);
    L.scount       = take(4 * (nB + 1));
    L.ecount       = take(4 * (nB + 1));
    L.unordered    = take(16);  // cleared together with the two count arrays before it
    L.state_off    = take(4 * (nB + 1));
    L.edge_off     = take(4 * (nB + 1));
    L.slot_off     = take(4 * (nB + 1));
    L.seq_T        = take(4 * nB);
    L.start_l      = take(4 * nB);
    L.end_l        = take(4 * nB);
    L.nslot        = take(4 * nB);
    L.ta_off       = take(8 * (nB + 1));
    L.tg_off       = take(8 * (nB + 1));
    L.gf_off       = take(8 * (nB + 1));
    L.gu_off       = take(8 * (nB + 1));
    L.pu_off       = take(8 * (nB + 1));
    L.order        = take(4 * nB);
    L.cost         = take(8 * nB);
    L.tx_off       = take(8 * (nB + 1));
    L.qpos         = take(4 * nE);
    L.m_pos        = take(8 * nE);
    L.eiota        = take(4 * nE);
    L.keyq         = take(4 * nE);
    L.keyf         = take(4 * nE);
    L.keyb         = take(4 * nE);
    L.key32_out    = take(4 * nE);
    L.qe           = take(4 * nE);
    L.fe           = take(4 * nE);
    L.be           = take(4 * nE);
    L.me           = take(4 * nE);
    L.slot_of_edge = take(4 * nE);
    L.key64        = take(8 * nE);
    L.key64_out    = take(8 * nE);
    L.head         = take(4 * (nE + 1));
    L.hs           = take(4 * (nE + 1));
    L.m_ptr        = take(4 * (nE + nB + 1));
    L.rowcnt_f     = take(4 * (nS + 1));
    L.rowptr_f     = take(4 * (nS + 1));
    L.rowcnt_b     = take(4 * (nS + 1));
    L.rowptr_b     = take(4 * (nS + 1));
    L.fwd_rec      = take(8 * nE);
    L.bwd_rec      = take(8 * nE);
    L.q_rec        = take(16 * nE);
    L.slot_emis    = take(4 * (nE + nB + 1));
    L.cub_temp_bytes = cub_temp_need(E, S);
    L.cub_temp       = take(L.cub_temp_bytes);
    L.total          = off;
    return L;
}

template <typename T>
T* at(void* base, size_t off) {
    return reinterpret_cast<T*>(reinterpret_cast<char*>(base) + off);
}
template <typename T>
const T* at(const void* base, size_t off) {
    return reinterpret_cast<const T*>(reinterpret_cast<const char*>(base) + off);
}

int bits_for(unsigned long long maxval) {
    int b = 1;
    while (b < 64 && (maxval >> b) != 0) b++;
    return b;
}

// ---------------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------------

// Log-semiring sum of two negative-log values; same expression as the reference's prob_add
// (i6_native_ops/fbw/fbw_op.cu:39-48) so results round identically.
__device__ __forceinline__ float prob_add(float a, float b) {
    float diff = a - b;
    if (isnan(diff)) {
        return CUDART_INF_F;
    }
    return -log1pf(expf(-fabsf(diff))) + fminf(a, b);
}

// prob_add with an exact shortcut.  prob_add(a,b) = fl(m - L), m = min(a,b), L = log1pf(expf(-d)),
// d = |a-b|.  L <= 2^(-d*log2(e)) (1 + 2^-20); if that is below a quarter of the smallest gap between
// m and a neighbouring float (2^(e-24) with e the exponent of m, taken at a power of two), the sum
// rounds back to m, so  d*log2(e) > 27 - e  implies the result is m bit for bit.  A NaN difference
// fails the test and takes the full path.
__device__ __forceinline__ bool prob_add_is_min(float a, float b, float m) {
    const float d = fabsf(a - b);
    const int   e = (int)((__float_as_uint(m) >> 23) & 0xffu) - 127;
    return d * 1.442695f > (float)(27 - e);
}

// first term of an accumulation that starts at +inf: prob_add(+inf, y) is y (or +inf for NaN)
__device__ __forceinline__ float prob_first(float y) { return isnan(y) ? CUDART_INF_F : y; }

// prob_add(acc, x) through the exact shortcuts: +inf terms, a first term, a provably dominated term
__device__ __forceinline__ float prob_add_fast(float acc, float x) {
    if (x == CUDART_INF_F) return acc;
    if (acc == CUDART_INF_F) return prob_first(x);
    const float m = fminf(acc, x);
    if (prob_add_is_min(acc, x, m)) return m;
    return prob_add(acc, x);
}

// prob_add(acc, x) with only the free shortcuts (+inf term, first term).  Used by the sweeps, where
// neighbouring states' scores are close and the dominance test rarely pays for itself.
__device__ __forceinline__ float prob_add_live(float acc, float x) {
    if (x == CUDART_INF_F) return acc;
    if (acc == CUDART_INF_F) return prob_first(x);
    return prob_add(acc, x);
}

// largest b in [0,B) with off[b] <= u, given off[0] <= u < off[B]
__device__ __forceinline__ int find_seq(const i64* __restrict__ off, int B, i64 u) {
    int lo = 0, hi = B;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (off[mid] <= u) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    return lo;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// prepare kernels
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ void claim_state(int* state_key, int* scount, int s, int q,
                                            fbw_b200_summary* hdr) {
    int old = atomicCAS(&state_key[s], -1, q);
    if (old == -1) {
        atomicAdd(&scount[q], 1);
    } else if (old != q) {
        atomicOr((unsigned long long*)&hdr->error, (unsigned long long)FBW_B200_ERR_SHARED_STATE);
    }
}

// start state of a plan in one launch: header and counters zero, no state owned yet
__global__ void k_init(fbw_b200_summary* hdr, int* state_key, i64 S, int* counters, i64 ncounters) {
    const i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < S) state_key[i] = -1;
    if (i < ncounters) counters[i] = 0;
    if (i < (i64)(sizeof(fbw_b200_summary) / sizeof(int64_t))) reinterpret_cast<int64_t*>(hdr)[i] = 0;
}

// one thread per edge, then one per sequence: range checks, edge counts, state ownership
__global__ void k_mark(const int* __restrict__ edges, const int* __restrict__ start_end, i64 E,
                       i64 B, i64 S, i64 F, int* state_key, int* scount, int* ecount,
                       int* unordered, fbw_b200_summary* hdr) {
    i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < E) {
        int fr = edges[idx], to = edges[E + idx], em = edges[2 * E + idx], sq = edges[3 * E + idx];
        // edges usually arrive sequence after sequence; then grouping them by sequence is the identity
        if (idx > 0 && sq < edges[3 * E + idx - 1]) unordered[0] = 1;
        unsigned long long err = 0;
        if (fr < 0 || fr >= S || to < 0 || to >= S) err |= FBW_B200_ERR_STATE_RANGE;
        if (em < 0 || em >= F) err |= FBW_B200_ERR_EMISSION_RANGE;
        if (sq < 0 || sq >= B) err |= FBW_B200_ERR_SEQ_RANGE;
        if (err) {
            atomicOr((unsigned long long*)&hdr->error, err);
            return;
        }
        {   // one atomic per group of lanes that share the sequence (edges usually arrive grouped)
            const unsigned peers = __match_any_sync(__activemask(), sq);
            if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&ecount[sq], __popc(peers));
        }
        claim_state(state_key, scount, fr, sq, hdr);
        claim_state(state_key, scount, to, sq, hdr);
    } else if (idx < E + B) {
        int b = (int)(idx - E);
        int s0 = start_end[b], s1 = start_end[B + b];
        if (s0 < 0 || s0 >= S || s1 < 0 || s1 >= S) {
            atomicOr((unsigned long long*)&hdr->error, (unsigned long long)FBW_B200_ERR_START_END);
            return;
        }
        claim_state(state_key, scount, s0, b, hdr);
        claim_state(state_key, scount, s1, b, hdr);
    }
}

// single block: exclusive scans of the per-sequence state and edge counts; effective lengths
__global__ void __launch_bounds__(1024) k_off1(const int* __restrict__ scount,
                                              const int* __restrict__ ecount,
                                              const int* __restrict__ seq_lens, int B, i64 T,
                                              int* state_off, int* edge_off, int* seq_T) {
    typedef cub::BlockScan<int, 1024> Scan;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ int carry[2];
    if (threadIdx.x == 0) carry[0] = carry[1] = 0;
    __syncthreads();
    for (int base = 0; base < B; base += 1024) {
        int  b  = base + threadIdx.x;
        bool ok = b < B;
        int  v[2] = {ok ? scount[b] : 0, ok ? ecount[b] : 0};
        int* dst[2] = {state_off, edge_off};
        for (int k = 0; k < 2; k++) {
            int ex, agg;
            Scan(tmp).ExclusiveSum(v[k], ex, agg);
            if (ok) dst[k][b] = carry[k] + ex;
            __syncthreads();
            if (threadIdx.x == 0) carry[k] += agg;
            __syncthreads();
        }
        if (ok) {
            // a sequence contributes only if 1 <= seq_len <= T: the backward seed is placed at
            // frame seq_len (fbw_op.cu:61-69 with the loop of 339-353), which never happens otherwise
            int n    = seq_lens[b];
            seq_T[b] = (n >= 1 && (i64)n <= T) ? n : 0;
        }
    }
    if (threadIdx.x == 0) {
        state_off[B] = carry[0];
        edge_off[B]  = carry[1];
    }
}

__global__ void k_statekeys(const int* __restrict__ state_key, i64 S, int B, unsigned* skey,
                            int* siota, int* unordered) {
    i64 s = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (s < S) {
        int k    = state_key[s];
        skey[s]  = k < 0 ? (unsigned)B : (unsigned)k;
        siota[s] = (int)s;
        // state ids usually run sequence after sequence (unused ids last); then ordering the states
        // by owning sequence is the identity
        if (s > 0) {
            const int kp = state_key[s - 1];
            if ((k < 0 ? B : k) < (kp < 0 ? B : kp)) unordered[1] = 1;
        }
    }
}

// Stable grouping of n items by key (a counting sort with known group offsets `off`), one CTA:
// perm[position] = item, inv[item] = position (inv may be null).  If the keys are already in
// non-decreasing order (*unordered == 0) the grouping is the identity and is written as such; that
// is the common case, and it replaces a device-wide radix sort (three kernels and two memsets) by
// one short kernel.  Otherwise the items are taken 1024 at a time, the warps of a chunk one after
// another, so that equal keys keep their order.
constexpr int kGroupKeys = 8192;
__global__ void __launch_bounds__(1024) k_group(const unsigned* __restrict__ keys, i64 n, int nkeys,
                                                const int* __restrict__ off,
                                                const int* __restrict__ unordered, int* perm, int* inv,
                                                const fbw_b200_summary* hdr) {
    __shared__ int cnt[kGroupKeys + 1];
    if (hdr->error) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (*unordered == 0) {
        for (i64 i = tid; i < n; i += 1024) {
            perm[i] = (int)i;
            if (inv) inv[i] = (int)i;
        }
        return;
    }
    for (int k = tid; k < nkeys; k += 1024) cnt[k] = 0;
    __syncthreads();
    for (i64 base = 0; base < n; base += 1024) {
        const i64  i  = base + tid;
        const bool in = i < n;
        const unsigned k = in ? keys[i] : 0xffffffffu;  // items past the end form a group of their own
        const unsigned peers = __match_any_sync(0xffffffffu, k);
        const int rank   = __popc(peers & ((1u << lane) - 1u));
        const int leader = __ffs(peers) - 1;
        int first = 0;
        for (int w = 0; w < 32; w++) {
            if (warp == w && in && lane == leader) {
                first = cnt[k];
                cnt[k] = first + __popc(peers);
            }
            __syncthreads();
        }
        first = __shfl_sync(0xffffffffu, first, leader);
        if (in) {
            const int pos = off[k] + first + rank;
            perm[pos] = (int)i;
            if (inv) inv[i] = pos;
        }
    }
}

__global__ void k_packed(const int* __restrict__ sorted_state, i64 S, int* packed_of) {
    i64 p = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (p < S) packed_of[sorted_state[p]] = (int)p;
}

__global__ void k_edgekeys(const int* __restrict__ edges, i64 E, i64 F,
                           const int* __restrict__ packed_of, unsigned* keyq, unsigned* keyf,
                           unsigned* keyb, unsigned long long* key64, int* eiota, int* rowcnt_f,
                           int* rowcnt_b, fbw_b200_summary* hdr) {
    if (hdr->error) return;
    i64 e = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (e < E) {
        int fr = edges[e], to = edges[E + e], em = edges[2 * E + e], sq = edges[3 * E + e];
        int pf = packed_of[fr], pt = packed_of[to];
        keyq[e]  = (unsigned)sq;
        keyf[e]  = (unsigned)pt;
        keyb[e]  = (unsigned)pf;
        key64[e] = (unsigned long long)sq * (unsigned long long)F + (unsigned long long)em;
        eiota[e] = (int)e;
        const int din  = atomicAdd(&rowcnt_f[pt], 1) + 1;
        const int dout = atomicAdd(&rowcnt_b[pf], 1) + 1;
        const int deg  = din > dout ? din : dout;
        // largest degree seen so far; the plain read keeps almost all edges off the atomic
        if ((i64)deg > *(volatile i64*)&hdr->max_degree) {
            atomicMax((unsigned long long*)&hdr->max_degree, (unsigned long long)deg);
        }
    }
}

__global__ void k_heads(const unsigned long long* __restrict__ key64s, i64 E, int* head) {
    i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < E) {
        head[i] = (i == 0 || key64s[i] != key64s[i - 1]) ? 1 : 0;
    } else if (i == E) {
        head[i] = 0;
    }
}

// hs[i] = number of class-group heads before position i of the (sequence, emission)-sorted list
__global__ void k_slots(const unsigned long long* __restrict__ key64s, const int* __restrict__ me,
                        const int* __restrict__ qe, const int* __restrict__ head,
                        const int* __restrict__ hs, i64 E, i64 F, int* slot_of_edge, int* slot_emis,
                        int* m_ptr, int* qpos, const fbw_b200_summary* hdr) {
    if (hdr->error) return;
    i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < E) {
        qpos[qe[i]] = (int)i;  // position of an edge in the sequence-grouped ascending list
        int g = hs[i] + head[i] - 1;  // global slot of this edge
        if (head[i]) {
            slot_emis[g] = (int)(key64s[i] % (unsigned long long)F);
            m_ptr[g]     = (int)i;
        }
        slot_of_edge[me[i]] = g;
    } else if (i == E) {
        m_ptr[hs[E]] = (int)E;
    }
}

// single block: everything per sequence that needs the slot counts.  Storage offsets of the run
// arrays are scans in sequence order; work-item offsets (gather and posterior units) are scans in
// RANK order, rank 0 being the most expensive sequence (frames x edges), so that kernels hand out
// work longest-first and a contiguous rank range is a group of similar cost.
__global__ void __launch_bounds__(1024) k_off2(const int* __restrict__ state_off,
                                              const int* __restrict__ edge_off,
                                              const int* __restrict__ hs,
                                              const int* __restrict__ seq_T,
                                              const int* __restrict__ start_end,
                                              const int* __restrict__ packed_of, int B, i64 T,
                                              i64 F, i64 E, i64 S, int* slot_off, int* nslot,
                                              int* start_l,
                                              int* end_l, i64* ta_off, i64* tg_off, i64* gf_off,
                                              i64* gu_off, i64* pu_off, i64* tx_off, i64* cost,
                                              int* order, int fast, fbw_b200_summary* hdr) {
    typedef cub::BlockScan<i64, 1024> Scan;
    __shared__ typename Scan::TempStorage tmp;
    __shared__ i64 carry[8];
    __shared__ int smax[4];
    __shared__ int smin;
    __shared__ int gmax[3][FBW_B200_GROUPS];
    if (threadIdx.x < 8) carry[threadIdx.x] = 0;
    if (threadIdx.x < 4) smax[threadIdx.x] = 0;
    if (threadIdx.x == 0) smin = 0x7fffffff;
    if (threadIdx.x < 3 * FBW_B200_GROUPS) (&gmax[0][0])[threadIdx.x] = 0;
    __syncthreads();
    const bool bad = hdr->error != 0;
    // ---- per sequence, sequence order: storage offsets, maxima, cost ----
    for (int base = 0; base < B; base += 1024) {
        int  b  = base + threadIdx.x;
        bool ok = b < B;
        i64  v[6] = {0, 0, 0, 0, 0, 0};
        if (ok) {
            int Sb = state_off[b + 1] - state_off[b];
            int Eb = edge_off[b + 1] - edge_off[b];
            // slot base and count: from the head scan (general path) or already written per
            // sequence by k_seqsort (fast path)
            int so = fast ? slot_off[b] : hs[edge_off[b]];
            int Db = fast ? nslot[b] : hs[edge_off[b + 1]] - so;
            int Te = seq_T[b];
            int nt = (Te + kTile - 1) / kTile;
            int Dp = (Db + 3) & ~3;
            slot_off[b] = so;
            nslot[b]    = Db;
            if (!bad) {
                start_l[b] = packed_of[start_end[b]] - state_off[b];
                end_l[b]   = packed_of[start_end[B + b]] - state_off[b];
            }
            v[0] = (i64)nt * Sb * kTile;
            v[1] = (i64)nt * Db * kTile;
            v[2] = (i64)Te * Dp;
            v[3] = Te;
            v[4] = (i64)nt * Eb * kTile;
            v[5] = Db;
            cost[b] = (i64)Te * (Eb + 1);
            atomicMax(&smax[0], Sb);
            atomicMax(&smax[1], Eb);
            atomicMax(&smax[2], Db);
            atomicMax(&smax[3], Te);
            if (Te > 0) atomicMin(&smin, Te);
        }
        i64* dst[6] = {ta_off, tg_off, gf_off, nullptr, tx_off, nullptr};
        for (int k = 0; k < 6; k++) {
            i64 ex, agg;
            Scan(tmp).ExclusiveSum(v[k], ex, agg);
            if (ok && dst[k]) dst[k][b] = carry[k] + ex;
            __syncthreads();
            if (threadIdx.x == 0) carry[k] += agg;
            __syncthreads();
        }
    }
    if (threadIdx.x == 0 && !fast) slot_off[B] = hs[E];
    __syncthreads();
    // ---- rank by descending cost (ties: ascending sequence id) ----
    for (int b = threadIdx.x; b < B; b += 1024) {
        const i64 cb = cost[b];
        int rank = 0;
        for (int j = 0; j < B; j++) {
            const i64 cj = cost[j];
            rank += (cj > cb || (cj == cb && j < b)) ? 1 : 0;
        }
        order[rank] = b;
    }
    __syncthreads();
    // ---- work-item offsets in rank order ----
    for (int base = 0; base < B; base += 1024) {
        int  r  = base + threadIdx.x;
        bool ok = r < B;
        i64  v[2] = {0, 0};
        if (ok) {
            int b  = order[r];
            int Db = nslot[b];
            int nt = (seq_T[b] + kTile - 1) / kTile;
            v[0] = (i64)nt * ((Db + kGatherSlots - 1) / kGatherSlots);
            v[1] = nt;
            int g = 0;  // group of rank r: groups are the rank ranges [g*B/G, (g+1)*B/G)
            for (int q = 1; q < FBW_B200_GROUPS; q++) {
                if (r >= (int)(((i64)q * B) / FBW_B200_GROUPS)) g = q;
            }
            atomicMax(&gmax[0][g], state_off[b + 1] - state_off[b]);
            atomicMax(&gmax[1][g], edge_off[b + 1] - edge_off[b]);
            atomicMax(&gmax[2][g], Db);
        }
        i64* dst[2] = {gu_off, pu_off};
        for (int k = 0; k < 2; k++) {
            i64 ex, agg;
            Scan(tmp).ExclusiveSum(v[k], ex, agg);
            if (ok) dst[k][r] = carry[6 + k] + ex;
            __syncthreads();
            if (threadIdx.x == 0) carry[6 + k] += agg;
            __syncthreads();
        }
    }
    if (threadIdx.x == 0) {
        ta_off[B] = carry[0];
        tg_off[B] = carry[1];
        gf_off[B] = carry[2];
        gu_off[B] = carry[6];
        pu_off[B] = carry[7];
        tx_off[B] = carry[4];
        hdr->score_floats = carry[4];
        hdr->T = T; hdr->B = B; hdr->F = F; hdr->E = E; hdr->S = S;
        hdr->state_floats = carry[0];
        hdr->tiled_floats = carry[1];
        hdr->frame_floats = carry[2];
        hdr->sum_len      = carry[3];
        hdr->gather_units = carry[6];
        hdr->post_units   = carry[7];
        hdr->num_slots    = carry[5];
        hdr->max_states = smax[0];
        hdr->max_edges  = smax[1];
        hdr->max_slots  = smax[2];
        hdr->max_len    = smax[3];
        hdr->min_len    = smin == 0x7fffffff ? 0 : smin;
        for (int g = 0; g < FBW_B200_GROUPS; g++) {
            hdr->group_max_states[g] = gmax[0][g];
            hdr->group_max_edges[g]  = gmax[1][g];
            hdr->group_max_slots[g]  = gmax[2][g];
        }
        if (smax[0] > kMaxPerSeq || smax[2] > kMaxPerSeq) {
            hdr->error |= FBW_B200_ERR_SEQ_TOO_LARGE;
        }
    }
}

// ---- fast path of prepare: one CTA sorts one sequence in shared memory --------------------------
constexpr int kFastThreads = 512;
constexpr int kFastItems   = 8;
constexpr int kFastCap     = kFastThreads * kFastItems;  // edges per sequence
constexpr int kFastPosBits = 12;                         // log2(kFastCap)

__global__ void k_seqkeys(const int* __restrict__ edges, i64 E, unsigned* keyq, int* eiota,
                          const fbw_b200_summary* hdr) {
    if (hdr->error) return;
    i64 e = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (e < E) {
        keyq[e]  = (unsigned)edges[3 * E + e];
        eiota[e] = (int)e;
    }
}

typedef cub::BlockRadixSort<unsigned, kFastThreads, kFastItems> FastSort;
typedef cub::BlockScan<int, kFastThreads>                       FastScan;
struct FastSmem {
    union {
        typename FastSort::TempStorage sort;
        typename FastScan::TempStorage scan;
    } t;
    unsigned sorted[kFastCap];     // the keys of the last sort, in order
    unsigned short from[kFastCap], to[kFastCap], slot[kFastCap];
    int      emis[kFastCap];
    unsigned last[kFastThreads];   // each thread's last sorted key (for the head test)
    int      deg_max;
};

// Builds everything the run kernels need for sequence b = blockIdx.x from the sequence-grouped edge
// list qe (ascending edge index inside the sequence): local slot numbers (distinct emissions in
// ascending order), the target-sorted and source-sorted edge lists with their row pointers, the
// emission-sorted list, all stable in edge index because the position in qe is the low part of every
// sort key.  Three block-wide radix sorts of at most 4096 keys replace three device-wide sorts.
__global__ void __launch_bounds__(kFastThreads) k_seqsort(
    const int* __restrict__ edges, const float* __restrict__ weights, i64 E, i64 F,
    const int* __restrict__ qe, const int* __restrict__ edge_off, const int* __restrict__ state_off,
    const int* __restrict__ packed_of, int* rowptr_f, int* rowptr_b, uint2* fwd_rec, uint2* bwd_rec,
    int4* q_rec, int2* m_pos, int* m_ptr, int* slot_emis, int* slot_off, int* nslot,
    fbw_b200_summary* hdr) {
    extern __shared__ __align__(16) unsigned char fast_raw[];
    FastSmem& sm = *reinterpret_cast<FastSmem*>(fast_raw);
    if (hdr->error & ~(i64)FBW_B200_ERR_RETRY_GENERAL) return;
    const int b = blockIdx.x, tid = threadIdx.x;
    const int e0 = edge_off[b], Eb = edge_off[b + 1] - e0;
    const int s0 = state_off[b], Sb = state_off[b + 1] - s0;
    const int so = e0 + b;  // base of this sequence's slot arrays (at most Eb slots, plus one end entry)
    if (tid == 0) slot_off[b] = so;
    if (Eb > kFastCap || F > (i64)(1u << (32 - kFastPosBits))) {
        if (tid == 0) {
            atomicOr((unsigned long long*)&hdr->error, (unsigned long long)FBW_B200_ERR_RETRY_GENERAL);
            nslot[b] = 0;
        }
        return;
    }
    if (tid == 0) sm.deg_max = 0;
    for (int i = tid; i < Eb; i += kFastThreads) {
        const int e = qe[e0 + i];
        sm.from[i] = (unsigned short)(packed_of[edges[e]] - s0);
        sm.to[i]   = (unsigned short)(packed_of[edges[E + e]] - s0);
        sm.emis[i] = edges[2 * E + e];
    }
    __syncthreads();
    const unsigned pos_mask = (1u << kFastPosBits) - 1u;
    unsigned keys[kFastItems];

    // ---- slots: sort by (emission, position) ----
#pragma unroll
    for (int k = 0; k < kFastItems; k++) {
        const int i = tid * kFastItems + k;
        keys[k] = i < Eb ? ((unsigned)sm.emis[i] << kFastPosBits) | (unsigned)i : 0xffffffffu;
    }
    FastSort(sm.t.sort).Sort(keys);
    sm.last[tid] = keys[kFastItems - 1];
    __syncthreads();
    int heads = 0;
    bool head[kFastItems];
#pragma unroll
    for (int k = 0; k < kFastItems; k++) {
        const int j = tid * kFastItems + k;
        const unsigned prev = k > 0 ? keys[k - 1] : (tid > 0 ? sm.last[tid - 1] : 0xffffffffu);
        head[k] = j < Eb && (j == 0 || (keys[k] >> kFastPosBits) != (prev >> kFastPosBits));
        heads += head[k] ? 1 : 0;
    }
    int before, total;
    FastScan(sm.t.scan).ExclusiveSum(heads, before, total);
    {
        int slot = before - 1;
#pragma unroll
        for (int k = 0; k < kFastItems; k++) {
            const int j = tid * kFastItems + k;
            if (j >= Eb) break;
            if (head[k]) {
                slot++;
                slot_emis[so + slot] = (int)(keys[k] >> kFastPosBits);
                m_ptr[so + slot]     = e0 + j;
            }
            const int i = (int)(keys[k] & pos_mask);
            sm.slot[i] = (unsigned short)slot;
            m_pos[e0 + j] = make_int2(i, slot);
        }
    }
    if (tid == 0) {
        m_ptr[so + total] = e0 + Eb;
        nslot[b]          = total;
    }
    __syncthreads();

    // ---- forward list (by target state) and backward list (by source state) ----
    for (int dir = 0; dir < 2; dir++) {
        const unsigned short* key_state = dir == 0 ? sm.to : sm.from;
        const unsigned short* other     = dir == 0 ? sm.from : sm.to;
        int*   rowptr = dir == 0 ? rowptr_f : rowptr_b;
        uint2* rec    = dir == 0 ? fwd_rec : bwd_rec;
#pragma unroll
        for (int k = 0; k < kFastItems; k++) {
            const int i = tid * kFastItems + k;
            keys[k] = i < Eb ? ((unsigned)key_state[i] << kFastPosBits) | (unsigned)i : 0xffffffffu;
        }
        __syncthreads();  // the previous use of the sort storage is over
        FastSort(sm.t.sort).Sort(keys);
#pragma unroll
        for (int k = 0; k < kFastItems; k++) {
            const int j = tid * kFastItems + k;
            sm.sorted[j] = keys[k];
            if (j < Eb) {
                const int i = (int)(keys[k] & pos_mask);
                rec[e0 + j] = make_uint2((unsigned)other[i] | ((unsigned)sm.slot[i] << 16),
                                         __float_as_uint(weights[qe[e0 + i]]));
            }
        }
        __syncthreads();
        // row pointers: first position whose state is >= s; the entry after the last state is the
        // first entry of the next sequence (both write the same value)
        int dmax = 0;
        for (int s = tid; s <= Sb; s += kFastThreads) {
            const unsigned want = (unsigned)s << kFastPosBits;
            int lo = 0, hi = Eb;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (sm.sorted[mid] < want) lo = mid + 1; else hi = mid;
            }
            rowptr[s0 + s] = e0 + lo;
            if (s < Sb) {
                const unsigned nxt = (unsigned)(s + 1) << kFastPosBits;
                int l2 = lo, h2 = Eb;
                while (l2 < h2) {
                    const int mid = (l2 + h2) >> 1;
                    if (sm.sorted[mid] < nxt) l2 = mid + 1; else h2 = mid;
                }
                dmax = max(dmax, l2 - lo);
            }
        }
        if (dmax > 0) atomicMax(&sm.deg_max, dmax);
        __syncthreads();
    }
    for (int i = tid; i < Eb; i += kFastThreads) {
        q_rec[e0 + i] = make_int4((int)sm.from[i], (int)sm.to[i], (int)sm.slot[i],
                                  __float_as_int(weights[qe[e0 + i]]));
    }
    if (tid == 0 && sm.deg_max > 0) {
        atomicMax((unsigned long long*)&hdr->max_degree, (unsigned long long)sm.deg_max);
    }
}

// the sorted edge lists as records with sequence-local state ids and class slots
__global__ void k_records(const int* __restrict__ edges, const float* __restrict__ weights, i64 E,
                          const int* __restrict__ packed_of, const int* __restrict__ state_off,
                          const int* __restrict__ slot_off, const int* __restrict__ slot_of_edge,
                          const int* __restrict__ qe, const int* __restrict__ fe,
                          const int* __restrict__ be, const int* __restrict__ me,
                          const int* __restrict__ qpos, const int* __restrict__ edge_off,
                          uint2* fwd_rec, uint2* bwd_rec, int4* q_rec, int2* m_pos,
                          const fbw_b200_summary* hdr) {
    if (hdr->error) return;
    i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= E) return;
    auto rec = [&](int e, int& fr, int& to, int& sl, float& w) {
        int sq = edges[3 * E + e];
        fr = packed_of[edges[e]] - state_off[sq];
        to = packed_of[edges[E + e]] - state_off[sq];
        sl = slot_of_edge[e] - slot_off[sq];
        w  = weights[e];
    };
    int   fr, to, sl;
    float w;
    rec(fe[i], fr, to, sl, w);
    fwd_rec[i] = make_uint2((unsigned)fr | ((unsigned)sl << 16), __float_as_uint(w));
    rec(be[i], fr, to, sl, w);
    bwd_rec[i] = make_uint2((unsigned)to | ((unsigned)sl << 16), __float_as_uint(w));
    rec(qe[i], fr, to, sl, w);
    q_rec[i] = make_int4(fr, to, sl, __float_as_int(w));
    rec(me[i], fr, to, sl, w);
    // (position in the sequence's ascending edge list, slot) for the class-posterior pass
    m_pos[i] = make_int2(qpos[me[i]] - edge_off[edges[3 * E + me[i]]], sl);
}

// ---------------------------------------------------------------------------------------------
// run kernels
// ---------------------------------------------------------------------------------------------
struct RunArgs {
    const float* am;
    float*       out;
    float*       sums;
    float*       loss2;
    float *A, *Bt, *Gt, *Gf, *P, *X, *N;
    const int *state_off, *edge_off, *slot_off, *nslot, *seq_T, *start_l, *end_l;
    const i64 *ta_off, *tg_off, *gf_off, *gu_off, *pu_off, *tx_off;
    const int2* m_pos;
    const int *rowptr_f, *rowptr_b;
    const uint2 *fwd_rec, *bwd_rec;
    const int4* q_rec;
    const int *m_ptr, *slot_emis, *order;
    i64 T, B, F;
    int r0, r1;  // rank range (a group of sequences) this launch works on
    // Time chunks: the sweeps advance chunk_steps frames per chunk from both ends of a sequence; a
    // launch handles the chunks [c_lo, c_hi).  One chunk covering everything is the plain case.
    int c_lo, c_hi, chunk_steps;
    float* carry;  // state vectors handed from one sweep chunk to the next, [2 * state][direction]
    // 1: the wrapper's passes are folded in -- `am` is log_probs (B,T,F) (sign and layout of the
    // caller's tensor, i6_native_ops/fbw/__init__.py:66) and `out` receives the gradient with respect
    // to it, -posterior in (B,T,F) with zeros elsewhere (what __init__.py:41-44 and autograd produce)
    int fused;
    // 1: `out` is pinned host memory the device writes over the bus; the output pass then stores its
    // segments with plain 16-byte vector stores instead of bulk copies from shared memory
    int out_plain;
    // 1: the sweeps compute every state's score, also of states that cannot lie on a complete path
    // (the debug export of the forward scores then equals the reference's buffer everywhere)
    int keep_dead_states;
    // Output in two steps (not null): the sweep launch of a group of sequences also writes the +inf
    // background of the group's rows of `out` -- one more warp per sweep CTA and `fill_ctas` CTAs that
    // do nothing else -- and k_patch writes the posteriors into it.  The word counts the rows taken.
    unsigned long long* next_row;
    int fill_ctas;
    int fill_piece;   // floats per bulk store of the background (a multiple of 32, at most kFillFloats)
    int fill_offset;  // where the block of background starts in the sweep CTA's dynamic shared memory (bytes)
    // 1: the frame-major score array Gf has been filled by the host (fbw_b200_run_with_host with scores in
    // host memory); k_gather then only builds the tiled copy from it
    int gathered_by_host;
};

// chunk in which the sweeps first need the scores of tile k of a sequence of Te frames: the forward
// sweep reaches frame 32k at step 32k, the backward sweep reaches the tile's last frame at step
// Te - 1 - last
__device__ __forceinline__ int tile_need_chunk(int k, int Te, int J) {
    const int last = min(k * kTile + kTile - 1, Te - 1);
    return min((k * kTile) / J, (Te - 1 - last) / J);
}
// chunk after which both alpha and beta of every frame of tile k are known: the forward sweep
// finishes the tile in the chunk of its last frame, the backward sweep in the chunk of step
// Te - 1 - 32k
__device__ __forceinline__ int tile_done_chunk(int k, int Te, int J) {
    const int last = min(k * kTile + kTile - 1, Te - 1);
    return max(last / J, (Te - 1 - k * kTile) / J);
}
__device__ __forceinline__ bool in_chunks(int c, const RunArgs& a) { return c >= a.c_lo && c < a.c_hi; }


// Gather am_scores[t,b,emission] for the distinct emissions ("slots", ascending emission id) of
// each sequence.  Work item = (sequence, 32-frame tile, 256 slots).  Two copies are written:
//   Gf  frame-major  [t][slot]           (rows padded to 4 floats)  -- read by the sweeps
//   Gt  tiled        [t/32][slot][t%32]                              -- read by k_post, lane = frame
__global__ void __launch_bounds__(256) k_gather(RunArgs a) {
    __shared__ float tile[kTile][kGatherSlots + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int B = (int)a.B;
    const i64 u_end = a.gu_off[a.r1];
    for (i64 u = a.gu_off[a.r0] + blockIdx.x; u < u_end; u += gridDim.x) {
        const int rk  = find_seq(a.gu_off, B, u);
        const int b   = a.order[rk];
        const int r   = (int)(u - a.gu_off[rk]);
        const int so  = a.slot_off[b];
        const int Db  = a.nslot[b];
        const int Dp  = (Db + 3) & ~3;
        const int nch = (Db + kGatherSlots - 1) / kGatherSlots;
        const int k = r / nch, c = r % nch;
        const int Te = a.seq_T[b];
        if (!in_chunks(tile_need_chunk(k, Te, a.chunk_steps), a)) continue;  // uniform in the CTA
        const int d0 = c * kGatherSlots;
        const int nd = min(kGatherSlots, Db - d0);
        const int* __restrict__ emis = a.slot_emis + so + d0;
        float* __restrict__ gf = a.Gf + a.gf_off[b];
        float* __restrict__ gt = a.Gt ? a.Gt + a.tg_off[b] + ((i64)k * Db + d0) * kTile : nullptr;

        int em[kGatherSlots / 32];
#pragma unroll
        for (int j = 0; j < kGatherSlots / 32; j++) {
            int dd = lane + 32 * j;
            em[j]  = dd < nd ? emis[dd] : 0;
        }
        for (int f = warp; f < kTile; f += 8) {
            const int  t     = k * kTile + f;
            const bool valid = t < Te;
            // (scores gathered by the host: the row of Gf itself, indexed by slot)
            const float* row = a.gathered_by_host
                                   ? gf + (i64)t * Dp + d0
                                   : a.am + (a.fused ? ((i64)b * a.T + t) : ((i64)t * B + b)) * a.F;
            const float sgn = a.fused == 1 ? -1.f : 1.f;  // 2: batch-major input, sign kept
            float v[kGatherSlots / 32];
#pragma unroll
            for (int j = 0; j < kGatherSlots / 32; j++) {
                int dd = lane + 32 * j;
                v[j]   = (valid && dd < nd) ? (a.gathered_by_host ? row[dd] : sgn * __ldg(row + em[j])) : CUDART_INF_F;
            }
#pragma unroll
            for (int j = 0; j < kGatherSlots / 32; j++) {
                int dd = lane + 32 * j;
                if (dd < nd) {
                    tile[f][dd] = v[j];
                    if (valid && !a.gathered_by_host) gf[(i64)t * Dp + d0 + dd] = v[j];
                }
            }
            if (valid && c == nch - 1 && !a.gathered_by_host) {
                for (int dd = Db + lane; dd < Dp; dd += 32) gf[(i64)t * Dp + dd] = 0.f;
            }
        }
        __syncthreads();
        if (gt) {
            for (int dd = warp; dd < nd; dd += 8) gt[(i64)dd * kTile + lane] = tile[lane][dd];
        }
        __syncthreads();
    }
}


// ---- the output in two steps: background with the sweeps, posteriors afterwards ---------------------
// Nearly all of the (T,B,F) output is the +inf background, which does not depend on anything the call
// computes, and the sweeps leave the memory system idle.  So the sweep launch of a group of sequences
// also writes the background of the group's rows: a warp of its own in every sweep CTA (and a few CTAs
// that do nothing else, for the SMs without a sweep) hands a constant block of +inf in shared memory
// to the copy engine over and over (cp.async.bulk shared -> global).  The block never changes, so no
// store waits for another, and the issue slots stay with the sweep.  Rows are handed out through a
// counter, so that every SM's copy engine is busy until the group's rows are done.  One warp per row;
// a row starts at any 4-byte offset: scalar head, 16-byte aligned body in pieces, scalar tail.
constexpr int kFillFloats = 2048;  // largest block of background in shared memory: 8 KB

__device__ __forceinline__ void sweep_sync(int nt) {  // the sweep's threads only (a multiple of 32)
    asm volatile("bar.sync 1, %0;" ::"r"(nt) : "memory");
}

__device__ __forceinline__ void background_rows(const RunArgs& a, const float* block) {
    // (`block` holds the background value of the mode: +inf, or 0 for the fused gradient output, whose
    // rows are ordered (sequence, frame))
    const float bg = a.fused ? 0.f : CUDART_INF_F;
    const int lane = threadIdx.x & 31;
    const int nb = a.r1 - a.r0;
    const i64 F = a.F;
    const i64 rows = a.T * nb;
    const unsigned src = (unsigned)__cvta_generic_to_shared(block);
    for (;;) {
        unsigned long long taken = 0;
        if (lane == 0) taken = atomicAdd(a.next_row, 1ull);
        const i64 it = (i64)__shfl_sync(0xffffffffu, taken, 0);
        if (it >= rows) break;
        const i64 t = it / nb;
        const int b = a.order[a.r0 + (int)(it - t * nb)];
        const i64 rbase = (a.fused ? (i64)b * a.T + t : t * a.B + b) * F;
        float* __restrict__ row = a.out + rbase;
        const int head = (int)min((i64)((4 - (rbase & 3)) & 3), F);
        const i64 body_end = head + (((F - head) >> 2) << 2);
        if (lane < head) row[lane] = bg;
        if (lane < F - body_end) row[body_end + lane] = bg;
        const i64 piece = a.fill_piece;
        for (i64 cs = head + (i64)lane * piece; cs < body_end; cs += 32 * piece) {
            const unsigned bytes = (unsigned)(min(piece, body_end - cs) * 4);
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(row + cs), "r"(src),
                         "r"(bytes)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        // a few stores in flight per lane: the next row is taken when the engine has room for it
        asm volatile("cp.async.bulk.wait_group 2;" ::: "memory");
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the block must outlive the stores
}

// One persistent CTA per (sequence, direction).  Shared memory holds the sequence's sorted edge list
// (target-sorted for the forward sweep, source-sorted for the backward one), the state-score
// vectors and a ring of RING gathered-score rows filled by cp.async a few frames ahead.
// Forward: alpha_0 = {start: 0}; alpha_{t+1}(s) = fold over in-edges, ascending edge index, of
// (alpha_t(from) + w) + score_t(emission).  alpha_t for t < len is stored (tiled) for k_post.
// Backward: beta_len = {end: 0}; beta_t(s) = fold over out-edges of (beta_{t+1}(to) + w) + score_t;
// the array stores beta_{t+1} at frame index t, which is what the edge score of frame t needs.
// TILED: the state vectors of the last 64 frames stay in shared memory and each finished 32-frame
// tile is written out as full 128-byte lines; otherwise every frame's vector is scattered out.
// Replaces set_start_states / init_bwd_state_buffer / next_frame / fill_array and the two host loops
// (fbw_op.cu:17-29, 61-102, 297-353).
// KREG: edges of a thread's state kept in registers (further edges are read from the list).
// prune != 0 (large automata): states that cannot lie on a complete path are skipped.  At set-up the
// CTA finds, by a breadth-first search over its edge list, the smallest number of frames each state
// needs to reach the sequence's end state (forward sweep) or to be reached from its start state
// (backward sweep).  A state that needs more frames than are left cannot lie on a path of exactly
// seq_len frames: its score can only ever meet a +inf score of the other direction in an edge score,
// so it is set to +inf without being computed.  The outputs are unchanged bit for bit; only the
// stored state scores of such dead states differ from the reference's forward buffer
// (RunArgs::keep_dead_states switches the skipping off for the debug export).  The states the sweep
// itself has not reached yet (+inf sources) are skipped edge by edge as before, so per frame only the
// band of states that are both reachable and useful costs arithmetic.
template <int RING, bool TILED, int KREG, bool PRUNE>
__global__ void __launch_bounds__(1024) k_sweep(RunArgs a, int smax, int dpmax, int edges_in_smem,
                                                int nrows) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int item = blockIdx.x;
    const int NT = blockDim.x - (a.next_row != nullptr ? 32 : 0);  // the sweep's threads
    if (a.next_row != nullptr) {
        const bool fill_only = item >= 2 * (a.r1 - a.r0);
        if (fill_only || (int)threadIdx.x >= NT) {
            // (the threads of a warp that writes the background all come here)
            // the block of background lies behind the sweep's own shared memory (launch_group)
            float* inf_block = reinterpret_cast<float*>(smem_raw + a.fill_offset);
            for (int i = (fill_only ? threadIdx.x : threadIdx.x - NT); i < a.fill_piece;
                 i += (fill_only ? blockDim.x : 32)) {
                inf_block[i] = a.fused ? 0.f : CUDART_INF_F;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (fill_only) __syncthreads(); else __syncwarp();
            background_rows(a, inf_block);
            return;
        }
    }
    const int b    = a.order[a.r0 + (item >> 1)];  // most expensive sequences first
    const bool fwd = (item & 1) == 0;
    const int  Te  = a.seq_T[b];
    if (Te == 0) return;
    const int s0 = a.state_off[b], Sb = a.state_off[b + 1] - s0;
    const int e0 = a.edge_off[b], Eb = a.edge_off[b + 1] - e0;
    const int Db = a.nslot[b];
    const int Dp = (Db + 3) & ~3;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = NT >> 5;
    // state vectors kept in shared memory: 64 (TILED), else nrows = 2 or 4.  With four, the vectors of
    // four consecutive frames leave as one 16-byte store per state instead of four 4-byte stores.
    const int kRows = TILED ? 64 : nrows;
    constexpr int kRegEdges = KREG;
    const int spad = TILED ? (smax | 1) : smax;  // odd row stride: conflict-free transposed reads

    float* ring  = reinterpret_cast<float*>(smem_raw);                      // RING * dpmax
    float* sbase = ring + (size_t)RING * dpmax;                             // kRows * spad
    int*   rp    = reinterpret_cast<int*>(sbase + (((size_t)kRows * spad + 3) & ~(size_t)3));
    unsigned short* hops = reinterpret_cast<unsigned short*>(rp + ((smax + 2) & ~1));  // if prune
    uint2* recs_s = reinterpret_cast<uint2*>(hops + ((smax + 3) & ~3));

    const int* __restrict__ rowptr = (fwd ? a.rowptr_f : a.rowptr_b) + s0;
    const uint2* __restrict__ recs_g = (fwd ? a.fwd_rec : a.bwd_rec) + e0;
    for (int s = tid; s <= Sb; s += NT) rp[s] = rowptr[s] - e0;
    const uint2* recs = recs_g;
    if (edges_in_smem) {
        for (int i = tid; i < Eb; i += NT) recs_s[i] = recs_g[i];
        recs = recs_s;
    }
    const bool prune = PRUNE && !a.keep_dead_states;
    if (prune) {
        // hops[s]: fewest frames from state s to the end state (forward sweep: the edge list is sorted
        // by target, so a settled state relaxes the sources of its in-edges) or from the start state
        // to s (backward sweep: list sorted by source, a settled state relaxes its targets).
        // Level-synchronous: one round per hop count, until a round settles nothing new.
        __shared__ int settled;
        const int far = 0xffff;
        const int origin = fwd ? a.end_l[b] : a.start_l[b];
        for (int s = tid; s < Sb; s += NT) hops[s] = (unsigned short)(s == origin ? 0 : far);
        sweep_sync(NT);
        for (int level = 0; level < far - 1; level++) {
            if (tid == 0) settled = 0;
            sweep_sync(NT);
            bool any = false;
            for (int s = tid; s < Sb; s += NT) {
                if (hops[s] == level) {
                    const int i1 = rp[s + 1];
                    for (int i = rp[s]; i < i1; i++) {
                        const int o = (int)(recs[i].x & 0xffffu);
                        if (hops[o] == far) {  // several writers may store the same value
                            hops[o] = (unsigned short)(level + 1);
                            any = true;
                        }
                    }
                }
            }
            if (any) settled = 1;
            sweep_sync(NT);
            if (settled == 0) break;  // uniform: read after the barrier, written before it
            sweep_sync(NT);
        }
    }
    const int step = fwd ? 1 : -1;
    const int t_first = fwd ? 0 : Te - 1;
    auto srow = [&](int j, int t) -> float* {
        return sbase + (size_t)(TILED ? (t & 63) : (j & (kRows - 1))) * spad;
    };
    // this launch covers steps [j0, j1) of the sequence's Te steps (a time chunk); a later chunk
    // picks up the state vector the previous one left in `carry`
    const int j0 = a.c_lo * a.chunk_steps;
    const int j1 = (int)min((i64)a.c_hi * a.chunk_steps, (i64)Te);
    if (j0 >= Te) return;
    float* __restrict__ carry = a.carry + 2 * (i64)s0 + (fwd ? 0 : Sb);
    {
        const int seed = fwd ? a.start_l[b] : a.end_l[b];
        float* r0 = srow(j0, t_first + step * j0);
        for (int s = tid; s < Sb; s += NT) {
            r0[s] = j0 == 0 ? ((s == seed) ? 0.f : CUDART_INF_F) : carry[s];
        }
    }
    sweep_sync(NT);
    // frames this launch records, for the tiled flush
    const int f_lo = fwd ? j0 : Te - j1, f_hi = fwd ? j1 - 1 : Te - 1 - j0;

    // the first state of this thread: its edges live in registers
    int   rfrom[kRegEdges], rslot[kRegEdges];
    float rw[kRegEdges];
    int   rcnt = 0, xi0 = 0, xi1 = 0;
    if (tid < Sb) {
        const int i0 = rp[tid], i1 = rp[tid + 1];
        rcnt = min(i1 - i0, kRegEdges);
        xi0  = i0 + rcnt;
        xi1  = i1;
#pragma unroll
        for (int k = 0; k < kRegEdges; k++) {
            const uint2 r = k < rcnt ? recs[i0 + k] : make_uint2(0u, __float_as_uint(CUDART_INF_F));
            rfrom[k] = (int)(r.x & 0xffffu);
            rslot[k] = (int)(r.x >> 16);
            rw[k]    = __uint_as_float(r.y);  // +inf for the entries past the state's edges
        }
    } else {
#pragma unroll
        for (int k = 0; k < kRegEdges; k++) { rfrom[k] = 0; rslot[k] = 0; rw[k] = CUDART_INF_F; }
    }

    const float* __restrict__ gf = a.Gf + a.gf_off[b];
    float* __restrict__ dst = (fwd ? a.A : a.Bt) + a.ta_off[b];
    const int nvec = Dp >> 2;
    // frames whose scores are consumed: forward 0..Te-2, backward Te-1..1
    auto issue = [&](int j) {  // j-th consumed frame
        if (RING > 0) {
            int t = t_first + step * j;
            if (j < Te - 1) {
                float*       d = ring + (size_t)(j % (RING > 0 ? RING : 1)) * dpmax;
                const float* g = gf + (i64)t * Dp;
                for (int i = tid; i < nvec; i += NT) cp_async16(d + 4 * i, g + 4 * i);
            }
            cp_async_commit();
        }
    };
    if (RING > 0) {
#pragma unroll
        for (int j = 0; j < RING - 1; j++) issue(j0 + j);
    }
    // write frames lo..hi (all inside tile k) of the shared-memory ring out as [state][32] lines
    auto flush_tile = [&](int k, int lo, int hi) {
        const int  frame = k * kTile + lane;
        const bool in    = frame >= lo && frame <= hi;
        const float* src = sbase + (size_t)(frame & 63) * spad;
        float* d = dst + (i64)k * Sb * kTile + lane;
        for (int s = warp; s < Sb; s += nwarps) {
            if (in) d[(i64)s * kTile] = src[s];
        }
    };

    constexpr int kWait = RING > 1 ? RING - 2 : 0;
    for (int j = j0; j < j1; j++) {
        const int t = t_first + step * j;
        if (RING > 0) cp_async_wait<kWait>();
        sweep_sync(NT);
        if (RING > 0) issue(j + RING - 1);
        const float* cur = srow(j, t);
        if (!TILED && kRows == 2) {  // record this frame's state scores (tiled layout: [t/32][state][t%32])
            float* drow = dst + ((i64)(t >> 5) * Sb) * kTile + (t & 31);
            for (int s = tid; s < Sb; s += NT) drow[(i64)s * kTile] = cur[s];
        } else if (!TILED) {
            // Four rows: the vectors of steps j-3 .. j are in shared memory.  When the sweep leaves an
            // aligned group of four frames (or the launch ends) the frames of that group recorded by
            // this launch are written, as one float4 per state if all four are there.  Every thread
            // reads only its own states' entries, which only itself overwrites (after this).
            const bool group_end  = fwd ? ((t & 3) == 3) : ((t & 3) == 0);
            const bool launch_end = j == j1 - 1;
            if (group_end || launch_end) {
                const int first = t_first + step * j0;  // first frame this launch recorded
                const int g0 = t & ~3;
                const int lo = fwd ? max(g0, first) : t;
                const int hi = fwd ? t : min(g0 + 3, first);
                float* base = dst + ((i64)(t >> 5) * Sb) * kTile + (g0 & 31);
                auto row_of = [&](int f) -> const float* {  // vector of frame f: step f or Te-1-f
                    return sbase + (size_t)((fwd ? f : Te - 1 - f) & 3) * spad;
                };
                if (lo == g0 && hi == g0 + 3) {
                    const float *r0 = row_of(g0), *r1 = row_of(g0 + 1), *r2 = row_of(g0 + 2), *r3 = row_of(g0 + 3);
                    for (int s = tid; s < Sb; s += NT) {
                        *reinterpret_cast<float4*>(base + (i64)s * kTile) = make_float4(r0[s], r1[s], r2[s], r3[s]);
                    }
                } else {
                    for (int f = lo; f <= hi; f++) {
                        const float* r = row_of(f);
                        for (int s = tid; s < Sb; s += NT) base[(i64)s * kTile + (f - g0)] = r[s];
                    }
                }
            }
        }
        const bool last  = j == Te - 1;           // the sequence ends here: nothing to compute
        const bool hand  = j == j1 - 1 && !last;  // a later chunk continues from the next vector
        if (!last) {
            float* nxt = srow(j + 1, t + step);
            const float* g = RING > 0 ? ring + (size_t)(j % (RING > 0 ? RING : 1)) * dpmax
                                      : gf + (i64)t * Dp;
            // frames left after this step for the state just computed: forward, alpha_{j+1} has
            // Te - (j+1) frames to reach the end; backward, beta at frame t must be reached from the
            // start in t frames.  A state that needs more is dead (see above).
            const int left = fwd ? Te - 1 - j : t;
            if (PRUNE && tid < Sb && prune && (int)hops[tid] > left) {
                nxt[tid] = CUDART_INF_F;
                if (hand) carry[tid] = CUDART_INF_F;
            } else if (tid < Sb) {
                // An unreachable source state (+inf) or a padding entry (weight +inf) gives +inf by
                // itself, and prob_add treats +inf terms exactly (a + inf term leaves the sum as it
                // is, a sum that is still +inf takes the term), so the register part needs no tests.
                float v[kRegEdges];
#pragma unroll
                for (int k = 0; k < kRegEdges; k++) v[k] = (cur[rfrom[k]] + rw[k]) + g[rslot[k]];
                float acc = prob_first(v[0]);
#pragma unroll
                for (int k = 1; k < kRegEdges; k++) acc = prob_add(acc, v[k]);
                for (int i = xi0; i < xi1; i++) {
                    const uint2 r  = recs[i];
                    const float pv = cur[r.x & 0xffffu];
                    if (!isinf(pv)) {
                        acc = prob_add_live(acc, (pv + __uint_as_float(r.y)) + g[r.x >> 16]);
                    }
                }
                nxt[tid] = acc;
                if (hand) carry[tid] = acc;
            }
            for (int s = tid + NT; s < Sb; s += NT) {
                float acc = CUDART_INF_F;
                const int i1 = (PRUNE && prune && (int)hops[s] > left) ? 0 : rp[s + 1];
                for (int i = rp[s]; i < i1; i++) {
                    const uint2 r  = recs[i];
                    const float pv = cur[r.x & 0xffffu];
                    if (!isinf(pv)) {
                        acc = prob_add_live(acc, (pv + __uint_as_float(r.y)) + g[r.x >> 16]);
                    }
                }
                nxt[s] = acc;
                if (hand) carry[s] = acc;
            }
        }
        if (TILED) {  // a tile is written when the sweep leaves it or the launch ends
            const int k = t >> 5;
            const bool out_now = fwd ? ((t & 31) == 31 || j == j1 - 1) : ((t & 31) == 0 || j == j1 - 1);
            if (out_now) flush_tile(k, max(k * kTile, f_lo), min(k * kTile + 31, f_hi));
        }
    }
    if (RING > 0) cp_async_wait<0>();
}

constexpr int kPostBatch = 8;  // edges whose lines are loaded together
// lines of edge scores a k_norm warp keeps in flight beyond the ones it is folding: the fold is a
// chain of dependent steps fed from DRAM, and its only parallelism is how far ahead it loads
constexpr int kNormBatch = 16;

// decode a work unit (sequence, 32-frame tile) from its index in rank order
struct PostUnit {
    int b, k, Sb, e0, Eb, so, Db, Dp, Te;
    i64 u;
};
__device__ __forceinline__ PostUnit post_unit(const RunArgs& a, i64 u) {
    PostUnit p;
    const int rk = find_seq(a.pu_off, (int)a.B, u);
    p.u  = u;
    p.b  = a.order[rk];
    p.k  = (int)(u - a.pu_off[rk]);
    p.Sb = a.state_off[p.b + 1] - a.state_off[p.b];
    p.e0 = a.edge_off[p.b];
    p.Eb = a.edge_off[p.b + 1] - p.e0;
    p.so = a.slot_off[p.b];
    p.Db = a.nslot[p.b];
    p.Dp = (p.Db + 3) & ~3;
    p.Te = a.seq_T[p.b];
    return p;
}

// Edge scores of every (frame, edge):
//   x_e = ((alpha_t(from) + w) + score_t(emission)) + beta_{t+1}(to)              (fbw_op.cu:93-100)
// written as X[tile][edge in ascending edge index][frame].  An unreachable source or target state
// has score +inf and so has the sum, which is what the reference stores for such an edge
// (fbw_op.cu:82-85).  One CTA per (sequence, 32-frame tile), lane = frame; in the tiled layouts
// every load and store of a warp is one 128-byte line.  Fully parallel: no fold here.
// (the work of `nwarps` warps on one unit; `warp` is this warp's number among them)
__device__ __forceinline__ void score_unit(const RunArgs& a, const PostUnit& p, int lane, int warp, int nwarps) {
    {
        const bool valid = p.k * kTile + lane < p.Te;
        // every lane loads (a tile is allocated for all 32 frames); frames past the sequence's
        // length hold unspecified values and get +inf
        const float* __restrict__ Ab = a.A + a.ta_off[p.b] + (i64)p.k * p.Sb * kTile + lane;
        const float* __restrict__ Bb = a.Bt + a.ta_off[p.b] + (i64)p.k * p.Sb * kTile + lane;
        const float* __restrict__ Gb = a.Gt + a.tg_off[p.b] + (i64)p.k * p.Db * kTile + lane;
        float* __restrict__ Xb = a.X + a.tx_off[p.b] + (i64)p.k * p.Eb * kTile + lane;
        const int4* __restrict__ q = a.q_rec + p.e0;
        for (int i0 = warp * kPostBatch; i0 < p.Eb; i0 += nwarps * kPostBatch) {
            int4  r[kPostBatch];
            float al[kPostBatch], be[kPostBatch], g[kPostBatch];
#pragma unroll
            for (int j = 0; j < kPostBatch; j++) r[j] = __ldg(q + min(i0 + j, p.Eb - 1));
#pragma unroll
            for (int j = 0; j < kPostBatch; j++) {
                al[j] = Ab[r[j].x * kTile];
                be[j] = Bb[r[j].y * kTile];
                g[j]  = Gb[r[j].z * kTile];
            }
#pragma unroll
            for (int j = 0; j < kPostBatch; j++) {
                const float v = ((al[j] + __int_as_float(r[j].w)) + g[j]) + be[j];
                if (i0 + j < p.Eb) Xb[(i64)(i0 + j) * kTile] = valid ? v : CUDART_INF_F;
            }
        }
    }
}

__global__ void __launch_bounds__(256) k_score(RunArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const i64 u0 = a.pu_off[a.r0], nunits = a.pu_off[a.r1] - u0;
    for (i64 idx = blockIdx.x; idx < nunits; idx += gridDim.x) {
        const PostUnit p = post_unit(a, u0 + idx);
        if (!in_chunks(tile_done_chunk(p.k, p.Te, a.chunk_steps), a)) continue;
        score_unit(a, p, lane, warp, 8);
    }
}

// Frame normalisers: sum = left fold of prob_add over the sequence's edges in ascending edge index
// (fbw_op.cu:115-118), sums[t,b] = isinf(sum) ? 0 : sum (fbw_op.cu:120-129).  One warp per
// (sequence, 32-frame tile), lane = frame, streaming the tile's edge scores in storage order; the
// next 8 lines are loaded while the current 8 are folded.  Steps whose result is provably the
// running minimum skip expf/log1pf (exact).  The raw sum (+inf for a dead frame) goes to N.
// Every unit is its own warp so that all the serial folds of a call run side by side.
// (one warp folds one unit; returns the raw sum of the lane's frame)
__device__ __forceinline__ float norm_unit(const RunArgs& a, const PostUnit& p, int lane) {
    {
        const int  t     = p.k * kTile + lane;
        const bool valid = t < p.Te;
        const float* __restrict__ Xb = a.X + a.tx_off[p.b] + (i64)p.k * p.Eb * kTile + lane;
        float acc = CUDART_INF_F;
        float nx[kNormBatch];
#pragma unroll
        for (int j = 0; j < kNormBatch; j++) nx[j] = j < p.Eb ? Xb[(i64)j * kTile] : CUDART_INF_F;
        for (int i0 = 0; i0 < p.Eb; i0 += kNormBatch) {
            float x[kNormBatch];
#pragma unroll
            for (int j = 0; j < kNormBatch; j++) x[j] = nx[j];
#pragma unroll
            for (int j = 0; j < kNormBatch; j++) {
                const int i = i0 + kNormBatch + j;
                nx[j] = i < p.Eb ? Xb[(i64)i * kTile] : CUDART_INF_F;
            }
#pragma unroll
            for (int j = 0; j < kNormBatch; j++) acc = prob_add_fast(acc, x[j]);
        }
        if (valid) a.sums[(i64)t * a.B + p.b] = isinf(acc) ? 0.f : acc;
        a.N[p.u * kTile + lane] = acc;
        return acc;
    }
}

__global__ void __launch_bounds__(128) k_norm(RunArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const i64 u0 = a.pu_off[a.r0], nunits = a.pu_off[a.r1] - u0;
    const i64 W = (i64)gridDim.x * 4;
    for (i64 idx = (i64)blockIdx.x * 4 + warp; idx < nunits; idx += W) {
        const PostUnit p = post_unit(a, u0 + idx);
        if (!in_chunks(tile_done_chunk(p.k, p.Te, a.chunk_steps), a)) continue;
        norm_unit(a, p, lane);
    }
}

// Class posteriors: post[t][slot] = -log sum over the slot's edges of exp(-(x_e - sum))
// (fbw_op.cu:131-153), as a running (minimum, scaled sum) pair.  The terms are normalised
// (magnitude of a log-posterior), so a fast exponential is accurate to ~1e-7 in the posterior; the
// reference accumulates the same terms with atomics in no fixed order.  A slot with one edge gets
// x_e - sum exactly.  One CTA per (sequence, 32-frame tile); each warp takes blocks of 32 slots,
// lane = frame, and writes them out transposed so that every frame's row of P is contiguous.
// (the work of `nwarps` warps on one unit; `st` is this warp's 32 x 33 staging tile, `acc` the raw
// sum of the lane's frame)
__device__ __forceinline__ void class_unit(const RunArgs& a, const PostUnit& p, int lane, int warp, int nwarps,
                                           float (*st)[kTile + 1], float acc) {
    {
        const bool rowdead = !(acc < CUDART_INF_F);  // no path through this frame
        const float* __restrict__ Xb = a.X + a.tx_off[p.b] + (i64)p.k * p.Eb * kTile + lane;
        const int2* __restrict__ m  = a.m_pos + p.e0;
        const int* __restrict__ mp  = a.m_ptr + p.so;
        float* __restrict__ Pb      = a.P + a.gf_off[p.b];
        const int mbase = mp[0];
        for (int d0 = warp * kTile; d0 < p.Db; d0 += nwarps * kTile) {
            const int nd = min(kTile, p.Db - d0);
            const int j0 = mp[d0] - mbase, j1 = mp[d0 + nd] - mbase;
            int   cur = -1;
            float mn = CUDART_INF_F, sme = 1.f;
            for (int i = j0; i < j1; i += kPostBatch) {
                int2  r[kPostBatch];
                float x[kPostBatch];
#pragma unroll
                for (int j = 0; j < kPostBatch; j++) r[j] = __ldg(m + min(i + j, j1 - 1));
#pragma unroll
                for (int j = 0; j < kPostBatch; j++) x[j] = Xb[(i64)r[j].x * kTile];
#pragma unroll
                for (int j = 0; j < kPostBatch; j++) {
                    if (i + j >= j1) continue;   // past the end of the block (uniform)
                    const float y = x[j] - acc;  // +inf for dead edges; NaN only if the row is dead
                    if (r[j].y != cur) {         // uniform: a new slot starts
                        if (cur >= 0) {
                            st[cur - d0][lane] =
                                (mn == CUDART_INF_F || rowdead) ? CUDART_INF_F : mn - logf(sme);
                        }
                        cur = r[j].y;
                        mn  = y;
                        sme = 1.f;
                    } else {
                        // running (minimum, sum scaled to it) without branches: the frames of a warp
                        // disagree on which term is the smaller, and both sides of a branch would run
                        const float nm = fminf(mn, y);
                        const float t1 = nm < CUDART_INF_F ? __expf(nm - mn) : 0.f;  // exp(-inf) = 0 while mn = +inf
                        const float t2 = y < CUDART_INF_F ? __expf(nm - y) : 0.f;
                        sme = sme * t1 + t2;
                        mn  = nm;
                    }
                }
            }
            if (cur >= 0) {
                st[cur - d0][lane] = (mn == CUDART_INF_F || rowdead) ? CUDART_INF_F : mn - logf(sme);
            }
            __syncwarp();
            // transpose: frame r of the tile gets its nd posteriors as one contiguous write
            for (int r = 0; r < kTile; r++) {
                const int tr = p.k * kTile + r;
                if (tr < p.Te && lane < nd) Pb[(i64)tr * p.Dp + d0 + lane] = st[lane][r];
            }
            __syncwarp();
        }
    }
}

constexpr int kClassWarps = 8;  // warps of a k_class CTA: blocks of 32 slots of one unit in flight
__global__ void __launch_bounds__(32 * kClassWarps) k_class(RunArgs a) {
    __shared__ float stage[kClassWarps][kTile][kTile + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const i64 u0 = a.pu_off[a.r0], nunits = a.pu_off[a.r1] - u0;
    for (i64 idx = blockIdx.x; idx < nunits; idx += gridDim.x) {
        const PostUnit p = post_unit(a, u0 + idx);
        if (!in_chunks(tile_done_chunk(p.k, p.Te, a.chunk_steps), a)) continue;
        class_unit(a, p, lane, warp, kClassWarps, stage[warp], a.N[p.u * kTile + lane]);
    }
}


// Stream the (T,B,F) output: every row is +inf except the sequence's class slots, which get the
// posteriors k_post left in P (frame-major, ascending emission id); rows at or past seq_len are all
// +inf.  One warp per row; the row is composed 512 floats at a time in shared memory and stored as
// 16-byte vectors.  Rows start at arbitrary 4-byte offsets (F need not be a multiple of 4), so each
// row is split into a scalar head, a 16-byte aligned body and a scalar tail.  One pass over the
// output instead of the reference's zeros_like + fill + atomics (fbw_op.cu:230, 366-378).
__global__ void __launch_bounds__(256) k_expand(RunArgs a) {
    __shared__ __align__(128) float segs[8][2][kSegFloats];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int B = (int)a.B;
    const i64 F = a.F;
    int which = 0;  // segment buffer in use; the other one may still be read by a store in flight
    // plain mode: background +inf, values are the negative log posteriors; fused mode: background 0,
    // values are -posterior (the gradient with respect to log_probs)
    const bool  fused = a.fused != 0;
    const float bg    = fused ? 0.f : CUDART_INF_F;
    auto pval = [&](float p) -> float { return fused ? -expf(-p) : p; };
    // Work item of a CTA: (32-frame tile, sequence), all T frames (frames past a sequence's length
    // are +inf rows).  A tile is written once the posteriors of its frames exist, i.e. in the chunk
    // after which both sweeps have passed it; tiles past the sequence's length go with chunk 0.
    const int nb  = a.r1 - a.r0;  // sequences of this group
    const int ntT = (int)((a.T + kTile - 1) / kTile);
    const i64 items = (i64)ntT * nb * 4;  // a work item per quarter tile (8 rows, one per warp)
    for (i64 it = blockIdx.x; it < items; it += gridDim.x) {
        const int  qt = (int)(it & 3);
        const i64  un = it >> 2;
        const int  k  = (int)(un / nb);
        const int  b  = a.order[a.r0 + (int)(un - (i64)k * nb)];
        {
            const int Te  = a.seq_T[b];
            const int dch = k * kTile < Te ? tile_done_chunk(k, Te, a.chunk_steps) : 0;
            if (!in_chunks(dch, a)) continue;  // uniform in the CTA
        }
        const int  t  = k * kTile + qt * 8 + warp;
        if (t >= a.T) continue;
        const i64  r  = a.fused ? (i64)b * a.T + t : (i64)t * B + b;
        const bool valid = t < a.seq_T[b];
        const int  so = a.slot_off[b];
        const int  Db = valid ? a.nslot[b] : 0;
        const int  Dp = (a.nslot[b] + 3) & ~3;
        const int* __restrict__ emis = a.slot_emis + so;
        const float* __restrict__ Pr = a.P + a.gf_off[b] + (i64)t * Dp;
        const i64 rbase = r * F;
        float* __restrict__ row = a.out + rbase;
        const int head = (int)min((i64)((4 - (rbase & 3)) & 3), F);
        const i64 nvec = (F - head) >> 2;
        const i64 body_end = head + 4 * nvec;

        int dlo = 0;  // next unconsumed slot; slots are in ascending emission id
        // head scalars
        if (head > 0) {
            float v = bg;
            // at most 3 columns: the first slots may fall here
            for (int d = 0; d < Db && d < 3; d++) {
                int e = emis[d];
                if (e == lane && e < head) v = pval(Pr[d]);
            }
            if (lane < head) row[lane] = v;
            while (dlo < Db && emis[dlo] < head) dlo++;
        }
        // aligned body: compose 512 floats in shared memory, hand them to the copy engine
        // (cp.async.bulk shared -> global), and compose the next segment in the other buffer
        // while that store is in flight
        for (i64 cs = head; cs < body_end; cs += kSegFloats) {
            const i64 ce = min(cs + (i64)kSegFloats, body_end);
            float* seg = segs[warp][which];
            // the store issued from this buffer two segments ago must have read it
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            {
                const float4 inf4 = make_float4(bg, bg, bg, bg);
                float4* s4 = reinterpret_cast<float4*>(seg);
#pragma unroll
                for (int i = 0; i < kSegFloats / 128; i++) s4[lane + 32 * i] = inf4;
            }
            __syncwarp();
            int n;
            if (Db * 8 > (int)F) {
                // a row dense in classes (lattices): many slots fall into one segment, and a loop
                // that loads 32 of them at a time is a chain of load latencies -- fetch four
                // batches ahead (slots are in ascending emission id, so a batch that does not lie
                // wholly in the segment ends the patching)
                do {
                    int   e[4];
                    float pv[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int d = dlo + 32 * q + lane;
                        e[q]  = d < Db ? emis[d] : 0x7fffffff;
                        pv[q] = d < Db ? Pr[d] : 0.f;
                    }
                    n = 32;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        if (n == 32) {  // uniform: every earlier batch lay wholly in the segment
                            const bool in = e[q] < ce;
                            if (in) seg[e[q] - cs] = pval(pv[q]);
                            n = __popc(__ballot_sync(0xffffffffu, in));
                            dlo += n;
                        }
                    }
                } while (n == 32);
            } else {
                do {  // patch the slots of this segment
                    const int d  = dlo + lane;
                    const int e  = d < Db ? emis[d] : 0x7fffffff;
                    const bool in = e < ce;
                    if (in) seg[e - cs] = pval(Pr[d]);
                    n = __popc(__ballot_sync(0xffffffffu, in));
                    dlo += n;
                } while (n == 32);
            }
            if (a.out_plain) {  // uniform: destination in host memory
                __syncwarp();
                const float4* s4 = reinterpret_cast<const float4*>(seg);
                float4* d4 = reinterpret_cast<float4*>(row + cs);
                const int nv = (int)((ce - cs) >> 2);
                for (int i = lane; i < nv; i += 32) d4[i] = s4[i];
                __syncwarp();
                which ^= 1;
                continue;
            }
            // make the generic-proxy writes visible to the async proxy, then one lane issues
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                const unsigned bytes = (unsigned)((ce - cs) * 4);
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(row + cs),
                             "r"((unsigned)__cvta_generic_to_shared(seg)), "r"(bytes)
                             : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            which ^= 1;
        }
        // tail scalars (at most 3 columns)
        {
            const int ntail = (int)(F - body_end);
            if (ntail > 0) {
                float v = bg;
                for (int d = dlo; d < Db; d++) {
                    if (emis[d] - body_end == lane) v = pval(Pr[d]);
                }
                if (lane < ntail) row[body_end + lane] = v;
            }
        }
    }
    // the buffers must outlive the stores that read them
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
}


// k_patch, the second step of the output in two steps (the first is background_rows, with the
// sweeps): the class posteriors go into rows that already hold the +inf background, as whole 32-byte
// sectors (the posterior and its +inf neighbours), which needs no read of the sector from DRAM; only
// the sectors that straddle two rows of the output are patched word by word.
// One warp per output row of a valid frame; lane = class slot.  A slot whose predecessor lies in
// another 32-byte sector leads its sector: it collects the posteriors of the slots that share the
// sector (slots are in ascending emission id, so they follow it) and writes the eight words.
__device__ __forceinline__ void patch_row(const RunArgs& a, const PostUnit& p, int t, int lane) {
    const int* __restrict__ emis = a.slot_emis + p.so;
    const float* __restrict__ Pr = a.P + a.gf_off[p.b] + (i64)t * p.Dp;
    const i64 F     = a.F;
    // plain mode: background +inf, values are the negative log posteriors; fused mode: background 0,
    // values are -posterior, rows ordered (sequence, frame) (see k_expand)
    const bool  fused = a.fused != 0;
    const float bg    = fused ? 0.f : CUDART_INF_F;
    const i64 rbase = (fused ? (i64)p.b * a.T + t : (i64)t * a.B + p.b) * F;  // first word of the row
    float* __restrict__ out = a.out;
    for (int d = lane; d < p.Db; d += 32) {
        const i64 g  = rbase + emis[d];
        const i64 sg = g >> 3;  // 32-byte sector of the output (out is 32-byte aligned)
        if (d > 0 && ((rbase + emis[d - 1]) >> 3) == sg) continue;  // not the first slot of its sector
        const i64 s0 = sg << 3;
        if (s0 >= rbase && s0 + 8 <= rbase + F) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = bg;
            for (int k = d; k < p.Db; k++) {
                const i64 gk = rbase + emis[k];
                if ((gk >> 3) != sg) break;
                const int pos = (int)(gk & 7);
                const float val = fused ? -expf(-Pr[k]) : Pr[k];
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = (i == pos) ? val : v[i];
            }
            float4* dst4 = reinterpret_cast<float4*>(out + s0);
            dst4[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst4[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {  // the sector holds words of a neighbouring row: patch this row's words one by one
            for (int k = d; k < p.Db; k++) {
                const i64 gk = rbase + emis[k];
                if ((gk >> 3) != sg) break;
                out[gk] = fused ? -expf(-Pr[k]) : Pr[k];
            }
        }
    }
}

__global__ void __launch_bounds__(256) k_patch(RunArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const i64 u0 = a.pu_off[a.r0], nunits = a.pu_off[a.r1] - u0;
    for (i64 idx = blockIdx.x; idx < nunits * 4; idx += gridDim.x) {  // a quarter tile (8 rows) per CTA step
        const PostUnit p = post_unit(a, u0 + (idx >> 2));
        if (!in_chunks(tile_done_chunk(p.k, p.Te, a.chunk_steps), a)) continue;
        const int t = p.k * kTile + (int)(idx & 3) * 8 + warp;
        if (t < p.Te) patch_row(a, p, t, lane);
    }
}

// Deterministic reduction of the per-frame sums into two scalars (single block).
__global__ void __launch_bounds__(1024) k_loss(const float* __restrict__ sums, i64 T, i64 B,
                                              float* loss2) {
    typedef cub::BlockReduce<double, 1024> Red;
    __shared__ typename Red::TempStorage tmp;
    double s_all = 0.0, s_first = 0.0;
    const i64 n = T * B;
    for (i64 i = threadIdx.x; i < n; i += 1024) {
        float v = sums[i];
        s_all += v;
        if (i < B) s_first += v;
    }
    double r0 = Red(tmp).Sum(s_all);
    __syncthreads();
    double r1 = Red(tmp).Sum(s_first);
    if (threadIdx.x == 0) {
        loss2[0] = (float)r0;
        loss2[1] = (float)r1;
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct RunLayout {
    size_t A, Bt, Gt, Gf, P, X, N, carry, next_row, total;
};

RunLayout run_layout(const fbw_b200_summary& s) {
    RunLayout L;
    size_t    off  = 0;
    auto      take = [&](size_t floats) {
        size_t o = off;
        off += ((floats + 8) * 4 + 255) & ~(size_t)255;  // slack: empty sequences read one float
        return o;
    };
    L.A     = take((size_t)s.state_floats);
    L.Bt    = take((size_t)s.state_floats);
    L.Gt    = take((size_t)s.tiled_floats);
    L.Gf    = take((size_t)s.frame_floats);
    L.P     = take((size_t)s.frame_floats);
    L.X     = take((size_t)s.score_floats);
    L.N     = take((size_t)s.post_units * kTile);
    L.carry = take((size_t)(2 * s.S));
    L.next_row = take(2 * FBW_B200_GROUPS);  // a 64-bit row counter per group (background_rows)
    L.total = off;
    return L;
}

// pinned host scratch of fbw_b200_run_with_host: the plan arrays the host threads read and the posteriors
struct HostLayout {
    size_t seq_T, nslot, slot_off, gf_off, slot_emis, P, G, total;
};

HostLayout host_layout(const fbw_b200_summary& s) {
    HostLayout H;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    H.seq_T     = take(4 * (size_t)s.B);
    H.nslot     = take(4 * (size_t)s.B);
    H.slot_off  = take(4 * (size_t)s.B);
    H.gf_off    = take(8 * (size_t)s.B);
    H.slot_emis = take(4 * (size_t)(s.E + s.B + 1));  // the plan's array: a sequence's classes start at slot_off[b] <= E
    H.P         = take(4 * ((size_t)s.frame_floats + 8));
    H.G         = take(4 * ((size_t)s.frame_floats + 8));  // scores gathered by the host
    H.total     = off;
    return H;
}

// the plan's arrays as kernel arguments: every sequence, one time chunk covering all frames
void plan_args(RunArgs& a, const void* plan, const fbw_b200_summary& s) {
    const PlanLayout L = plan_layout(s.B, s.E, s.S);
    a.state_off = at<int>(plan, L.state_off);
    a.edge_off  = at<int>(plan, L.edge_off);
    a.slot_off  = at<int>(plan, L.slot_off);
    a.nslot     = at<int>(plan, L.nslot);
    a.seq_T     = at<int>(plan, L.seq_T);
    a.start_l   = at<int>(plan, L.start_l);
    a.end_l     = at<int>(plan, L.end_l);
    a.ta_off = at<i64>(plan, L.ta_off);
    a.tg_off = at<i64>(plan, L.tg_off);
    a.gf_off = at<i64>(plan, L.gf_off);
    a.gu_off = at<i64>(plan, L.gu_off);
    a.pu_off = at<i64>(plan, L.pu_off);
    a.tx_off = at<i64>(plan, L.tx_off);
    a.m_pos  = at<int2>(plan, L.m_pos);
    a.rowptr_f = at<int>(plan, L.rowptr_f);
    a.rowptr_b = at<int>(plan, L.rowptr_b);
    a.fwd_rec  = at<uint2>(plan, L.fwd_rec);
    a.bwd_rec  = at<uint2>(plan, L.bwd_rec);
    a.q_rec    = at<int4>(plan, L.q_rec);
    a.m_ptr     = at<int>(plan, L.m_ptr);
    a.slot_emis = at<int>(plan, L.slot_emis);
    a.order     = at<int>(plan, L.order);
    a.T = s.T; a.B = s.B; a.F = s.F;
    a.r0 = 0; a.r1 = (int)s.B;
    a.c_lo = 0; a.c_hi = 1; a.chunk_steps = 1 << 30;
    a.next_row = nullptr;
    a.fill_ctas = 0;
    a.fill_piece = kFillFloats;
    a.fill_offset = 0;
    a.gathered_by_host = 0;
}

// the arguments of one forward-backward call: plan arrays, run scratch, inputs and outputs
RunArgs fbw_args(const void* plan, const fbw_b200_summary& s, void* work, const RunLayout& R,
                 const float* am, float* out, float* sums, float* loss2, int fused) {
    RunArgs a;
    memset(&a, 0, sizeof(a));
    plan_args(a, plan, s);
    a.am = am; a.out = out; a.sums = sums; a.loss2 = loss2;
    a.A  = at<float>(work, R.A);
    a.Bt = at<float>(work, R.Bt);
    a.Gt = at<float>(work, R.Gt);
    a.Gf = at<float>(work, R.Gf);
    a.P  = at<float>(work, R.P);
    a.X  = at<float>(work, R.X);
    a.N  = at<float>(work, R.N);
    a.carry = at<float>(work, R.carry);
    a.fused = fused;
    return a;
}

// largest per-group maxima of a plan: what a launch over all sequences has to be sized for
void plan_maxima(const fbw_b200_summary& s, i64& ms, i64& me, i64& md) {
    ms = me = md = 0;
    for (int q = 0; q < FBW_B200_GROUPS; q++) {
        ms = s.group_max_states[q] > ms ? s.group_max_states[q] : ms;
        me = s.group_max_edges[q] > me ? s.group_max_edges[q] : me;
        md = s.group_max_slots[q] > md ? s.group_max_slots[q] : md;
    }
}

constexpr int kMaxDevices = 64;

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    return dev;
}

// SM count of the current device (asked once per device)
int sm_count() {
    static std::atomic<int> n[kMaxDevices];
    const int dev = current_device();
    int v = n[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
            v = 148;
        }
        n[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

// Raise a kernel's dynamic shared-memory limit to `smem` bytes unless an earlier launch on this
// device already raised it that far (`granted` is the per-device record of one kernel).
template <typename Kernel>
cudaError_t grant_smem(Kernel kernel, std::atomic<int>* granted, size_t smem) {
    if (smem <= 48 * 1024) return cudaSuccess;
    const int dev = current_device();
    if ((size_t)granted[dev].load(std::memory_order_relaxed) >= smem) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) granted[dev].store((int)smem, std::memory_order_relaxed);
    return e;
}

std::atomic<long long> g_launches{0};
#define COUNT_LAUNCH(n) g_launches.fetch_add((n), std::memory_order_relaxed)

#define CUDA_OK(expr)                            \
    do {                                         \
        if ((expr) != cudaSuccess) {             \
            return FBW_B200_CUDA_ERROR;          \
        }                                        \
    } while (0)

template <int RING, bool TILED, int KREG, bool PRUNE>
int launch_sweep_k(const RunArgs& a, int grid, int nt, size_t smem, int smax, int dpmax,
                   int edges_in_smem, int nrows, cudaStream_t st) {
    static std::atomic<int> granted[kMaxDevices];
    CUDA_OK(grant_smem(k_sweep<RING, TILED, KREG, PRUNE>, granted, smem));
    k_sweep<RING, TILED, KREG, PRUNE><<<grid, nt, smem, st>>>(a, smax, dpmax, edges_in_smem, nrows);
    COUNT_LAUNCH(1);
    return FBW_B200_OK;
}

template <int RING, bool TILED>
int launch_sweep(const RunArgs& a, int grid, int nt, size_t smem, int smax, int dpmax,
                 int edges_in_smem, int nrows, int degree, cudaStream_t st) {
    // skipping dead states pays for its set-up where a state has many edges or a thread several states
    static int forced = -1;
    if (forced < 0) { const char* e = getenv("FBW_B200_PRUNE"); forced = e ? atoi(e) : 2; }
    const int prune = forced == 2 ? (degree >= 6 ? 1 : 0) : forced;
    // (the pruning variant exists for the four-register kernel only: automata with at most three
    // edges per state are chains, where almost every state is alive almost all of the time)
    if (degree <= 2) return launch_sweep_k<RING, TILED, 2, false>(a, grid, nt, smem, smax, dpmax, edges_in_smem, nrows, st);
    if (degree <= 3) return launch_sweep_k<RING, TILED, 3, false>(a, grid, nt, smem, smax, dpmax, edges_in_smem, nrows, st);
    if (prune) return launch_sweep_k<RING, TILED, 4, true>(a, grid, nt, smem, smax, dpmax, edges_in_smem, nrows, st);
    return launch_sweep_k<RING, TILED, 4, false>(a, grid, nt, smem, smax, dpmax, edges_in_smem, nrows, st);
}

#include "sweep_cluster_b200.inc"
// CTAs per cluster for the sweeps of `items` (sequence, direction) pairs of automata of at most ms
// states, when `spare` SMs would otherwise stay idle during the call's sweeps.  A cluster spreads the
// per-frame work of one large sequence over several SMs, which shortens the call only while SMs are
// free: a call that already has a sweep CTA for every SM gains nothing and pays for the cluster
// barriers.  Returns 1, 2 or 4 and takes the SMs it uses off `spare`.  FBW_B200_CLUSTER=1|2|4 fixes
// the answer.
int sweep_cluster_size(i64 ms, int items, int* spare) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("FBW_B200_CLUSTER");
        forced = e ? atoi(e) : 0;
    }
    if (forced == 1 || forced == 2 || forced == 4) return forced;
    if (ms <= 1024 || items <= 0) return 1;
    for (int cs = ms > 2048 ? 4 : 2; cs > 1; cs >>= 1) {
        const int extra = (cs - 1) * items;
        if (extra <= *spare) {
            *spare -= extra;
            return cs;
        }
    }
    return 1;
}

constexpr int kMaxChunks = 16;
constexpr int kPostStreams = 4;  // aux[1..4] carry the output stages, aux[0] the gather

// streams and events for the per-group pipelines, one pool per device, created on first use
struct StreamPool {
    std::mutex   mu;
    bool         ready = false, failed = false;
    cudaStream_t aux[FBW_B200_GROUPS];
    cudaStream_t copy;  // device -> host copies of finished parts of the output
    cudaEvent_t  fork, join[FBW_B200_GROUPS], copied;
    // fbw_b200_run_with_host: one such call per device at a time (its thread waits on these events)
    std::mutex   host_mu;
    cudaEvent_t  host_ready, host_done[kMaxChunks];
    cudaEvent_t  gathered[kMaxChunks], swept[kMaxChunks], expanded[kMaxChunks];
};
StreamPool g_pools[kMaxDevices];
std::mutex g_pools_mu;

StreamPool* stream_pool() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    StreamPool* p = &g_pools[dev];
    std::lock_guard<std::mutex> lk(g_pools_mu);
    if (p->failed) return nullptr;
    if (!p->ready) {
        bool ok = cudaEventCreateWithFlags(&p->fork, cudaEventDisableTiming) == cudaSuccess &&
                  cudaEventCreateWithFlags(&p->copied, cudaEventDisableTiming) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&p->copy, cudaStreamNonBlocking) == cudaSuccess;
        for (int i = 0; i < FBW_B200_GROUPS && ok; i++) {
            ok = cudaStreamCreateWithFlags(&p->aux[i], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&p->join[i], cudaEventDisableTiming) == cudaSuccess;
        }
        ok = ok && cudaEventCreateWithFlags(&p->host_ready, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; i < kMaxChunks && ok; i++) {
            ok = cudaEventCreateWithFlags(&p->host_done[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&p->gathered[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&p->swept[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&p->expanded[i], cudaEventDisableTiming) == cudaSuccess;
        }
        if (!ok) {
            p->failed = true;
            return nullptr;
        }
        p->ready = true;
    }
    return p;
}

// number of size groups (1 or 8): batches whose largest automaton is several times the average, and
// large batches in general
int choose_groups(const fbw_b200_summary& s) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("FBW_B200_NUM_GROUPS");
        forced = e ? atoi(e) : 0;
    }
    if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return s.B >= forced ? forced : 1;
    // Batches with large automata (more states than a sweep CTA has threads: lattices) run as groups at
    // every batch size: groups give each range of the cost order its own launch shape and cluster size,
    // which the time-chunk pipeline cannot (lattice, ms per call, time chunks against four groups: 8
    // sequences 7.9 / 6.6, 24: 20.3 / 11.4, 48: 26.7 / 13.0).  Four groups up to about 70 sequences (64:
    // 13.7 ms against 14.9 with eight), eight beyond (80: 14.7 against 18.3 with four).
    if (s.B >= 4 && s.max_states > 1024) return s.B >= 72 ? 8 : 4;
    if (s.B >= 64 && s.E > 0 && (double)s.max_edges * (double)s.B >= 1.8 * (double)s.E &&
        s.max_edges >= 2048) {
        return 8;
    }
    // Large calls whose sweep CTAs (two per sequence) fill the machine also run as groups: every
    // group's gather is an eighth of the whole, so the first sweeps start early, and the output
    // stages of the groups that finish first overlap with the sweeps of the others.  (Measured on
    // the triphone workload: B = 64 2.59 ms against 2.68 ms for the time-chunk pipeline, B = 128 4.53
    // against 4.94; with B = 32 or 16 the time chunks win, 1.86 against 2.05 and 1.53 against 1.62.)
    const double cells = (double)s.T * (double)s.B * (double)s.F;
    if (cells >= 1.0e8 && 2 * s.B >= (i64)sm_count() * 4 / 5) return 8;
    return 1;
}

// number of time chunks of the pipeline: small calls run as one chunk on the caller's stream
int choose_chunks(const fbw_b200_summary& s) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("FBW_B200_NUM_CHUNKS");
        forced = e ? atoi(e) : 0;
    }
    int C = 1;
    const double cells = (double)s.T * (double)s.B * (double)s.F;
    if (cells >= 1.0e8 && s.max_len >= 512) C = 6;
    if (forced >= 1) C = forced;
    if (C > kMaxChunks) C = kMaxChunks;
    while (C > 1 && s.max_len / C < 2 * kTile) C--;  // at least two tiles per chunk
    return C;
}

// Launch shape of k_sweep for automata of at most ms states, me edges and md class slots.
// Shared memory of the kernel: score ring, state rows (64 tiled, else 4 or 2), row pointers, edge
// records.  Preference: edges in shared memory, then tiled state rows, then a score ring with four
// state rows, a ring with two, and last no ring at all.
struct SweepShape {
    bool   found;
    int    ring, tiled, rows, in_smem, smax, dpmax, nt;
    size_t smem;
};
SweepShape sweep_shape(i64 ms, i64 me, i64 md) {
    SweepShape c;
    c.found = false;
    c.ring = c.tiled = c.in_smem = 0;
    c.rows = 2;
    c.smem  = 0;
    c.smax  = (int)((ms + 3) & ~3);
    c.dpmax = (int)((md + 3) & ~3);
    c.nt    = (int)((ms + 31) & ~31);
    c.nt    = c.nt < 64 ? 64 : (c.nt > 1024 ? 1024 : c.nt);
    const size_t limit = 227 * 1024 - sizeof(float) * kFillFloats - 128;  // room for the block of background
    auto need = [&](int ring, int rows, int in_smem) {
        const size_t spad = rows == 64 ? (size_t)(c.smax | 1) : (size_t)c.smax;
        return (size_t)4 * ring * c.dpmax + 4 * (((size_t)rows * spad + 3) & ~(size_t)3) +
               (size_t)4 * ((c.smax + 2) & ~1) + (size_t)2 * ((c.smax + 3) & ~3) +
               (in_smem ? (size_t)8 * me : 0) + 16;
    };
    static int rows4 = -1;
    if (rows4 < 0) { const char* e = getenv("FBW_B200_ROWS4"); rows4 = e ? atoi(e) : 1; }
    for (int es = 1; es >= 0 && !c.found; es--) {
        // pass 0: 64 rows; 1: 4 rows with a ring; 2: 2 rows with a ring; 3: 4 rows, no ring; 4: 2 rows, no ring
        for (int pass = 0; pass < 5 && !c.found; pass++) {
            const int rows = pass == 0 ? 64 : ((pass == 1 || pass == 3) ? 4 : 2);
            if (rows == 4 && !rows4) continue;
            for (int rg = (pass >= 3 ? 0 : 16); rg >= (pass >= 3 || pass == 0 ? 0 : 2) && !c.found; rg = rg > 2 ? rg / 2 : rg - 2) {
                if (need(rg, rows, es) <= limit) {
                    c.ring = rg; c.tiled = rows == 64; c.rows = rows; c.in_smem = es; c.found = true;
                    c.smem = need(rg, rows, es);
                }
            }
        }
    }
    return c;
}

// Whether a call that runs as groups writes its output in two steps (background_rows with the sweeps,
// k_patch after the posteriors) instead of one pass of k_expand afterwards.  It pays where the rows
// are sparse (the sectors that hold a posterior are a small part of the row) and the background does
// not hold up the sweeps: all sweep CTAs resident at once, or a background that takes longer than the
// sweeps anyway.  Measured, ms per call, one pass against two steps: triphone 64 sequences 2.55 / 2.40,
// 96 sequences 3.43 / 3.72 (sweep CTAs in two waves: the first wave leaves later), BPE-CTC 256
// sequences 1.49 / 1.30, 128 sequences 1.06 / 0.90.  FBW_B200_OUTPUT=patch / expand fixes the answer.
bool output_in_two_steps(const fbw_b200_summary& s, i64 ms, i64 me, i64 md) {
    static int conf = -1;
    if (conf < 0) {
        const char* e = getenv("FBW_B200_OUTPUT");
        conf = e && strcmp(e, "patch") == 0 ? 1 : (e && strcmp(e, "expand") == 0 ? 0 : 2);
    }
    // the sweep CTAs need room for one more warp; automata that large run as clusters anyway
    if (conf == 0 || s.max_len <= 0 || ms > 992) return false;
    const SweepShape c = sweep_shape(ms, me, md);
    if (!c.found) return false;
    if (conf == 1) return true;
    if (md * 16 > s.F) return false;  // dense rows: patching would touch most sectors twice
    const i64 by_smem    = (i64)(227 * 1024) / (i64)(c.smem + sizeof(float) * 512 + 128 + 1024);
    const i64 by_threads = 2048 / (c.nt + 32);
    const i64 per_sm     = by_smem < by_threads ? (by_smem > 0 ? by_smem : 1) : (by_threads > 0 ? by_threads : 1);
    const i64 waves      = (2 * s.B + per_sm * sm_count() - 1) / (per_sm * sm_count());
    if (waves <= 1) return true;
    const double fill_ms  = (double)s.T * (double)s.B * (double)s.F * 4.0 / 5.0e9;  // at 5 TB/s
    const double sweep_ms = (double)waves * (double)s.max_len * 0.6e-3;             // 0.6 us per frame
    return fill_ms >= 1.3 * sweep_ms;
}

// gather -> sweep -> posterior -> expand for the sequences of ranks [r0, r1) on stream st.
// ms/me/md: largest state, edge and slot counts in the range (they size the sweep launch).
enum { kDoGather = 1, kDoSweep = 2, kDoPost = 4, kDoExpand = 8, kDoAll = 15, kDoPatch = 16 };

// `what` selects the stages to launch (the time-chunked pipeline launches them on different streams)
int launch_group(RunArgs a, int r0, int r1, i64 ms, i64 me, i64 md, const fbw_b200_summary& s,
                 cudaStream_t st, cudaEvent_t* ev, int what = kDoAll, int cs = 1) {
    const int sms = sm_count();
    const int nb  = r1 - r0;
    a.r0 = r0;
    a.r1 = r1;
    const i64 tiles = (s.max_len + kTile - 1) / kTile;
    if (ev) CUDA_OK(cudaEventRecord(ev[0], st));
    if ((what & kDoGather) && s.gather_units > 0 && md > 0) {
        i64 want = tiles * nb * ((md + kGatherSlots - 1) / kGatherSlots);
        int grid = (int)(want < (i64)sms * 6 ? want : (i64)sms * 6);
        k_gather<<<grid > 0 ? grid : 1, 256, 0, st>>>(a);
        COUNT_LAUNCH(1);
    }
    if (ev) CUDA_OK(cudaEventRecord(ev[1], st));
    if ((what & kDoSweep) && s.max_len > 0 && cs > 1 && cluster_shape(ms, me, md, cs).found) {
        const int rc = launch_sweepc(a, cluster_shape(ms, me, md, cs), 2 * nb, st);
        if (rc != FBW_B200_OK) return rc;
    } else if ((what & kDoSweep) && s.max_len > 0) {
        const SweepShape c = sweep_shape(ms, me, md);
        if (!c.found) return FBW_B200_TOO_LARGE;
        const int smax = c.smax, dpmax = c.dpmax, nt = c.nt, ring = c.ring, tiled = c.tiled;
        const int in_smem = c.in_smem;
        // with the background: its block behind the sweep's shared memory, a warp more per CTA, and CTAs
        // that do nothing else
        size_t smem = c.smem;
        if (a.next_row != nullptr) {
            a.fill_offset = (int)((c.smem + 127) & ~(size_t)127);
            smem = (size_t)a.fill_offset + sizeof(float) * (size_t)a.fill_piece;
        }
        const int grid = 2 * nb + (a.next_row != nullptr ? a.fill_ctas : 0);
        const int nthreads = nt + (a.next_row != nullptr ? 32 : 0);
        int rc;
#define SWEEP_CASE(R, TL) \
    rc = launch_sweep<R, TL>(a, grid, nthreads, smem, smax, dpmax, in_smem, c.rows, (int)s.max_degree, st)
        if (tiled) {
            switch (ring) {
                case 16: SWEEP_CASE(16, true); break;
                case 8: SWEEP_CASE(8, true); break;
                case 4: SWEEP_CASE(4, true); break;
                case 2: SWEEP_CASE(2, true); break;
                default: SWEEP_CASE(0, true); break;
            }
        } else {
            switch (ring) {
                case 16: SWEEP_CASE(16, false); break;
                case 8: SWEEP_CASE(8, false); break;
                case 4: SWEEP_CASE(4, false); break;
                case 2: SWEEP_CASE(2, false); break;
                default: SWEEP_CASE(0, false); break;
            }
        }
#undef SWEEP_CASE
        if (rc != FBW_B200_OK) return rc;
    }
    if (ev) CUDA_OK(cudaEventRecord(ev[2], st));
    if ((what & kDoPost) && s.post_units > 0) {
        const i64 units = tiles * nb;  // upper bound; the kernels read the exact count
        int g1 = (int)(units < (i64)sms * 8 ? units : (i64)sms * 8);
        i64 w2 = (units + 3) / 4;
        int g2 = (int)(w2 < (i64)sms * 16 ? w2 : (i64)sms * 16);
        int g3 = (int)(units < (i64)sms * 6 ? units : (i64)sms * 6);
        k_score<<<g1 > 0 ? g1 : 1, 256, 0, st>>>(a);
        k_norm<<<g2 > 0 ? g2 : 1, 128, 0, st>>>(a);
        k_class<<<g3 > 0 ? g3 : 1, 32 * kClassWarps, 0, st>>>(a);
        COUNT_LAUNCH(3);
    }
    if (ev) CUDA_OK(cudaEventRecord(ev[3], st));
    if (what & kDoPatch) {
        const i64 want = tiles * nb * 4;
        int grid = (int)(want < (i64)sms * 8 ? want : (i64)sms * 8);
        k_patch<<<grid > 0 ? grid : 1, 256, 0, st>>>(a);
        COUNT_LAUNCH(1);
    }
    if (what & kDoExpand) {
        i64 want = ((s.T + kTile - 1) / kTile) * nb * 4;
        int grid = (int)(want < (i64)sms * 8 ? want : (i64)sms * 8);
        k_expand<<<grid, 256, 0, st>>>(a);
        COUNT_LAUNCH(1);
    }
    return FBW_B200_OK;
}

}  // namespace

extern "C" {

int fbw_b200_abi_version(void) { return 4; }

const char* fbw_b200_status_string(int status) {
    switch (status) {
        case FBW_B200_OK: return "ok";
        case FBW_B200_BAD_ARGUMENT: return "bad argument (null pointer, non-positive dimension or misaligned buffer)";
        case FBW_B200_WORKSPACE: return "workspace too small";
        case FBW_B200_CUDA_ERROR: return "CUDA runtime error";
        case FBW_B200_BAD_AUTOMATON: return "automaton rejected (index out of range, state shared by two sequences, or a sequence too large)";
        case FBW_B200_TOO_LARGE: return "request exceeds the fixed capacity of this entry point";
        case FBW_B200_RETRY_GENERAL: return "plan must be rebuilt with fbw_b200_prepare_general";
        default: return "unknown status";
    }
}

size_t fbw_b200_plan_bytes(int64_t B, int64_t E, int64_t S) {
    if (B <= 0 || S <= 0 || E < 0) return 0;
    return plan_layout(B, E, S).total;
}

static int prepare_impl(const int32_t* edges, const float* weights, const int32_t* start_end,
                        const int32_t* seq_lens, int64_t T, int64_t B, int64_t F, int64_t E,
                        int64_t S, void* plan, size_t plan_bytes, fbw_b200_stream_t stream,
                        bool allow_fast) {
    if (T <= 0 || B <= 0 || F <= 0 || S <= 0 || E < 0) return FBW_B200_BAD_ARGUMENT;
    if (B > 0x7fffffff / 2 || E > 0x7fffffff - 1 || S > 0x7fffffff - 1 || T > 0x7fffffff)
        return FBW_B200_BAD_ARGUMENT;
    if (!plan || !start_end || !seq_lens || (E > 0 && (!edges || !weights)))
        return FBW_B200_BAD_ARGUMENT;
    if (((uintptr_t)plan & 255) != 0) return FBW_B200_BAD_ARGUMENT;
    const PlanLayout L = plan_layout(B, E, S);
    if (plan_bytes < L.total) return FBW_B200_WORKSPACE;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

    // Fast path: the edges are grouped by sequence with one device-wide sort and every sequence is
    // then sorted three ways by one CTA in shared memory (k_seqsort).  It needs every sequence to
    // have at most kFastCap edges; the host can only judge the average, a sequence over the limit
    // flags the plan for a retry through the general path.
    const bool fast = allow_fast && E > 0 && E / B <= kFastCap / 2 && F <= (i64)(1u << (32 - kFastPosBits));

    fbw_b200_summary* hdr = at<fbw_b200_summary>(plan, L.header);
    {   // header, state owners, and the counters scount / ecount / unordered (one contiguous range)
        const i64 ncounters = (i64)((L.state_off - L.scount) / 4);
        const i64 n = S > ncounters ? S : ncounters;
        k_init<<<(unsigned)((n + 255) / 256 > 0 ? (n + 255) / 256 : 1), 256, 0, st>>>(
            hdr, at<int>(plan, L.state_key), S, at<int>(plan, L.scount), ncounters);
        COUNT_LAUNCH(1);
    }
    if (!fast) {
        CUDA_OK(cudaMemsetAsync(at<int>(plan, L.rowcnt_f), 0, 4 * (size_t)(S + 1), st));
        CUDA_OK(cudaMemsetAsync(at<int>(plan, L.rowcnt_b), 0, 4 * (size_t)(S + 1), st));
        CUDA_OK(cudaMemsetAsync(at<int>(plan, L.hs), 0, 4 * (size_t)(E + 1), st));
        CUDA_OK(cudaMemsetAsync(at<int>(plan, L.m_ptr), 0, 4 * (size_t)(E + B + 1), st));
    }

    const int TB = 256;
    auto blocks = [&](i64 n) { return (unsigned)((n + TB - 1) / TB); };
    void*  ctemp = at<char>(plan, L.cub_temp);
    size_t cbytes = L.cub_temp_bytes;

    COUNT_LAUNCH(fast ? 7 : (E > 0 ? 9 : 5));  // k_mark, k_off1, k_statekeys, k_packed, k_off2 + edge kernels
    int* unordered = at<int>(plan, L.unordered);
    // grouping by sequence with one CTA instead of a device-wide sort (see k_group)
    const bool group1 = fast && B < kGroupKeys;
    k_mark<<<blocks(E + B), TB, 0, st>>>(edges, start_end, E, B, S, F, at<int>(plan, L.state_key),
                                         at<int>(plan, L.scount), at<int>(plan, L.ecount), unordered,
                                         hdr);
    k_off1<<<1, 1024, 0, st>>>(at<int>(plan, L.scount), at<int>(plan, L.ecount), seq_lens, (int)B,
                               T, at<int>(plan, L.state_off), at<int>(plan, L.edge_off),
                               at<int>(plan, L.seq_T));
    // states ordered by owning sequence (stable: ascending state id inside a sequence)
    k_statekeys<<<blocks(S), TB, 0, st>>>(at<int>(plan, L.state_key), S, (int)B,
                                          at<unsigned>(plan, L.skey), at<int>(plan, L.siota),
                                          unordered);
    if (group1) {
        // keys 0..B (B = state id not used by any sequence), group offsets = state_off[0..B]
        k_group<<<1, 1024, 0, st>>>(at<unsigned>(plan, L.skey), S, (int)B + 1,
                                    at<int>(plan, L.state_off), unordered + 1,
                                    at<int>(plan, L.sorted_state), at<int>(plan, L.packed_of), hdr);
    } else {
        CUDA_OK(cub::DeviceRadixSort::SortPairs(ctemp, cbytes, at<unsigned>(plan, L.skey),
                                                at<unsigned>(plan, L.skey_out),
                                                at<int>(plan, L.siota), at<int>(plan, L.sorted_state),
                                                (int)S, 0, bits_for((unsigned long long)B), st));
        k_packed<<<blocks(S), TB, 0, st>>>(at<int>(plan, L.sorted_state), S, at<int>(plan, L.packed_of));
    }
    if (fast) {
        if (group1) {
            // the sequence ids of the edges are the keys (validated by k_mark, which flags the plan
            // otherwise), group offsets = edge_off
            k_group<<<1, 1024, 0, st>>>(reinterpret_cast<const unsigned*>(edges + 3 * E), E, (int)B,
                                        at<int>(plan, L.edge_off), unordered, at<int>(plan, L.qe),
                                        nullptr, hdr);
        } else {
            k_seqkeys<<<blocks(E), TB, 0, st>>>(edges, E, at<unsigned>(plan, L.keyq),
                                                at<int>(plan, L.eiota), hdr);
            CUDA_OK(cub::DeviceRadixSort::SortPairs(ctemp, cbytes, at<unsigned>(plan, L.keyq),
                                                    at<unsigned>(plan, L.key32_out),
                                                    at<int>(plan, L.eiota), at<int>(plan, L.qe), (int)E,
                                                    0, bits_for((unsigned long long)B), st));
        }
        static std::atomic<int> granted[kMaxDevices];
        CUDA_OK(grant_smem(k_seqsort, granted, sizeof(FastSmem)));
        k_seqsort<<<(unsigned)B, kFastThreads, sizeof(FastSmem), st>>>(
            edges, weights, E, F, at<int>(plan, L.qe), at<int>(plan, L.edge_off),
            at<int>(plan, L.state_off), at<int>(plan, L.packed_of), at<int>(plan, L.rowptr_f),
            at<int>(plan, L.rowptr_b), at<uint2>(plan, L.fwd_rec), at<uint2>(plan, L.bwd_rec),
            at<int4>(plan, L.q_rec), at<int2>(plan, L.m_pos),
            at<int>(plan, L.m_ptr), at<int>(plan, L.slot_emis), at<int>(plan, L.slot_off),
            at<int>(plan, L.nslot), hdr);
    } else if (E > 0) {
        k_edgekeys<<<blocks(E), TB, 0, st>>>(edges, E, F, at<int>(plan, L.packed_of),
                                             at<unsigned>(plan, L.keyq), at<unsigned>(plan, L.keyf),
                                             at<unsigned>(plan, L.keyb),
                                             at<unsigned long long>(plan, L.key64),
                                             at<int>(plan, L.eiota), at<int>(plan, L.rowcnt_f),
                                             at<int>(plan, L.rowcnt_b), hdr);
        const int sb = bits_for((unsigned long long)S);
        CUDA_OK(cub::DeviceRadixSort::SortPairs(ctemp, cbytes, at<unsigned>(plan, L.keyq),
                                                at<unsigned>(plan, L.key32_out),
                                                at<int>(plan, L.eiota), at<int>(plan, L.qe), (int)E,
                                                0, bits_for((unsigned long long)B), st));
        CUDA_OK(cub::DeviceRadixSort::SortPairs(ctemp, cbytes, at<unsigned>(plan, L.keyf),
                                                at<unsigned>(plan, L.key32_out),
                                                at<int>(plan, L.eiota), at<int>(plan, L.fe), (int)E,
                                                0, sb, st));
        CUDA_OK(cub::DeviceRadixSort::SortPairs(ctemp, cbytes, at<unsigned>(plan, L.keyb),
                                                at<unsigned>(plan, L.key32_out),
                                                at<int>(plan, L.eiota), at<int>(plan, L.be), (int)E,
                                                0, sb, st));
        CUDA_OK(cub::DeviceRadixSort::SortPairs(
            ctemp, cbytes, at<unsigned long long>(plan, L.key64),
            at<unsigned long long>(plan, L.key64_out), at<int>(plan, L.eiota), at<int>(plan, L.me),
            (int)E, 0, bits_for((unsigned long long)B * (unsigned long long)F), st));
        CUDA_OK(cub::DeviceScan::ExclusiveSum(ctemp, cbytes, at<int>(plan, L.rowcnt_f),
                                              at<int>(plan, L.rowptr_f), (int)(S + 1), st));
        CUDA_OK(cub::DeviceScan::ExclusiveSum(ctemp, cbytes, at<int>(plan, L.rowcnt_b),
                                              at<int>(plan, L.rowptr_b), (int)(S + 1), st));
        k_heads<<<blocks(E + 1), TB, 0, st>>>(at<unsigned long long>(plan, L.key64_out), E,
                                              at<int>(plan, L.head));
        CUDA_OK(cub::DeviceScan::ExclusiveSum(ctemp, cbytes, at<int>(plan, L.head),
                                              at<int>(plan, L.hs), (int)(E + 1), st));
        k_slots<<<blocks(E + 1), TB, 0, st>>>(at<unsigned long long>(plan, L.key64_out),
                                              at<int>(plan, L.me), at<int>(plan, L.qe),
                                              at<int>(plan, L.head), at<int>(plan, L.hs), E, F,
                                              at<int>(plan, L.slot_of_edge),
                                              at<int>(plan, L.slot_emis), at<int>(plan, L.m_ptr),
                                              at<int>(plan, L.qpos), hdr);
    } else {
        CUDA_OK(cudaMemsetAsync(at<int>(plan, L.rowptr_f), 0, 4 * (size_t)(S + 1), st));
        CUDA_OK(cudaMemsetAsync(at<int>(plan, L.rowptr_b), 0, 4 * (size_t)(S + 1), st));
    }
    k_off2<<<1, 1024, 0, st>>>(at<int>(plan, L.state_off), at<int>(plan, L.edge_off),
                               at<int>(plan, L.hs), at<int>(plan, L.seq_T), start_end,
                               at<int>(plan, L.packed_of), (int)B, T, F, E, S,
                               at<int>(plan, L.slot_off), at<int>(plan, L.nslot),
                               at<int>(plan, L.start_l),
                               at<int>(plan, L.end_l), at<i64>(plan, L.ta_off),
                               at<i64>(plan, L.tg_off), at<i64>(plan, L.gf_off),
                               at<i64>(plan, L.gu_off), at<i64>(plan, L.pu_off),
                               at<i64>(plan, L.tx_off), at<i64>(plan, L.cost),
                               at<int>(plan, L.order), fast ? 1 : 0, hdr);
    if (E > 0 && !fast) {
        k_records<<<blocks(E), TB, 0, st>>>(
            edges, weights, E, at<int>(plan, L.packed_of), at<int>(plan, L.state_off),
            at<int>(plan, L.slot_off), at<int>(plan, L.slot_of_edge), at<int>(plan, L.qe),
            at<int>(plan, L.fe), at<int>(plan, L.be), at<int>(plan, L.me), at<int>(plan, L.qpos),
            at<int>(plan, L.edge_off), at<uint2>(plan, L.fwd_rec), at<uint2>(plan, L.bwd_rec),
            at<int4>(plan, L.q_rec), at<int2>(plan, L.m_pos), hdr);
    }
    CUDA_OK(cudaGetLastError());
    return FBW_B200_OK;
}

int fbw_b200_prepare(const int32_t* edges, const float* weights, const int32_t* start_end,
                     const int32_t* seq_lens, int64_t T, int64_t B, int64_t F, int64_t E, int64_t S,
                     void* plan, size_t plan_bytes, fbw_b200_stream_t stream) {
    return prepare_impl(edges, weights, start_end, seq_lens, T, B, F, E, S, plan, plan_bytes, stream,
                        true);
}

int fbw_b200_prepare_general(const int32_t* edges, const float* weights, const int32_t* start_end,
                             const int32_t* seq_lens, int64_t T, int64_t B, int64_t F, int64_t E,
                             int64_t S, void* plan, size_t plan_bytes, fbw_b200_stream_t stream) {
    return prepare_impl(edges, weights, start_end, seq_lens, T, B, F, E, S, plan, plan_bytes, stream,
                        false);
}

int fbw_b200_plan_summary(const void* plan, fbw_b200_summary* summary, fbw_b200_stream_t stream) {
    if (!plan || !summary) return FBW_B200_BAD_ARGUMENT;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    CUDA_OK(cudaMemcpyAsync(summary, plan, sizeof(fbw_b200_summary), cudaMemcpyDeviceToHost, st));
    CUDA_OK(cudaStreamSynchronize(st));
    if (summary->error == FBW_B200_ERR_RETRY_GENERAL) return FBW_B200_RETRY_GENERAL;
    return summary->error ? FBW_B200_BAD_AUTOMATON : FBW_B200_OK;
}

size_t fbw_b200_run_bytes(const fbw_b200_summary* summary) {
    if (!summary) return 0;
    return run_layout(*summary).total;
}

// The plan arrays the host threads read, copied into the pinned scratch behind `st` (complete when
// `ready` has happened), and `h` pointed at them.
static int host_plan_arrays(const void* plan, const fbw_b200_summary& s, char* hw, const HostLayout& H,
                            cudaStream_t st, cudaEvent_t ready, fbw_b200::HostRows& h) {
    const PlanLayout L = plan_layout(s.B, s.E, s.S);
    CUDA_OK(cudaMemcpyAsync(hw + H.seq_T, at<int>(plan, L.seq_T), 4 * (size_t)s.B, cudaMemcpyDeviceToHost, st));
    CUDA_OK(cudaMemcpyAsync(hw + H.nslot, at<int>(plan, L.nslot), 4 * (size_t)s.B, cudaMemcpyDeviceToHost, st));
    CUDA_OK(cudaMemcpyAsync(hw + H.slot_off, at<int>(plan, L.slot_off), 4 * (size_t)s.B, cudaMemcpyDeviceToHost, st));
    CUDA_OK(cudaMemcpyAsync(hw + H.gf_off, at<i64>(plan, L.gf_off), 8 * (size_t)s.B, cudaMemcpyDeviceToHost, st));
    CUDA_OK(cudaMemcpyAsync(hw + H.slot_emis, at<int>(plan, L.slot_emis), 4 * (size_t)(s.E + s.B + 1),
                            cudaMemcpyDeviceToHost, st));
    CUDA_OK(cudaEventRecord(ready, st));
    h.T = s.T; h.B = s.B; h.F = s.F;
    h.seq_T     = reinterpret_cast<const int*>(hw + H.seq_T);
    h.nslot     = reinterpret_cast<const int*>(hw + H.nslot);
    h.slot_off  = reinterpret_cast<const int*>(hw + H.slot_off);
    h.gf_off    = reinterpret_cast<const int64_t*>(hw + H.gf_off);
    h.slot_emis = reinterpret_cast<const int*>(hw + H.slot_emis);
    h.P   = nullptr;
    h.out = nullptr;
    h.am  = nullptr;
    h.batch_major = 0;
    h.chunk_steps = 1 << 30;
    h.first_chunk = 0;
    h.num_slots = s.E + s.B + 1;
    h.p_floats  = s.frame_floats;
    return FBW_B200_OK;
}

static int run_impl(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                    float* sums, float* loss2, void* work, size_t work_bytes,
                    fbw_b200_stream_t stream, cudaEvent_t* ev, int fused = 0, int keep_dead_states = 0,
                    float* out_host = nullptr, void* host_work = nullptr, bool host_writes_rows = false) {
    // host_work (fbw_b200_run_with_host): pinned host scratch; host threads of the library take over what
    // is slow over the bus (host_fill.cpp).  Scores in host memory: they pick the scores the automata
    // need out of the tensor.  host_writes_rows (sparse rows): `out` IS a pinned host buffer and no
    // kernel composes rows; the class posteriors go to pinned host memory as the posterior stages
    // finish, and the host threads write the rows from them while the device goes on.
    const bool host_help  = host_work != nullptr;
    const bool host_patch = host_help && host_writes_rows;
    if (!plan || !summary || !am || !out || !sums || !work) return FBW_B200_BAD_ARGUMENT;
    if (summary->error) return FBW_B200_BAD_AUTOMATON;
    if (((uintptr_t)out & 15) != 0 || ((uintptr_t)work & 255) != 0) return FBW_B200_BAD_ARGUMENT;
    const fbw_b200_summary& s = *summary;
    const RunLayout  R = run_layout(s);
    if (work_bytes < R.total) return FBW_B200_WORKSPACE;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    RunArgs a = fbw_args(plan, s, work, R, am, out, sums, loss2, fused);
    a.keep_dead_states = keep_dead_states;
    fbw_b200::HostRows host_rows;
    const HostLayout H = host_layout(s);
    StreamPool* host_pool = host_help ? stream_pool() : nullptr;
    std::unique_lock<std::mutex> host_lock;
    int  host_first_chunk = 0, host_chunks = 0;
    if (host_help) {
        if (fused || out_host) return FBW_B200_BAD_ARGUMENT;
        if (!host_pool) return FBW_B200_CUDA_ERROR;
        host_lock = std::unique_lock<std::mutex>(host_pool->host_mu);
        // the little the host has to know about the plan, and the posteriors' place in host memory
        char* hw = static_cast<char*>(host_work);
        const int rc = host_plan_arrays(plan, s, hw, H, st, host_pool->host_ready, host_rows);
        if (rc != FBW_B200_OK) return rc;
        if (host_patch) a.P = reinterpret_cast<float*>(hw + H.P);
        host_rows.P   = a.P;
        host_rows.out = out;
    }
    const int host_nthreads = host_help ? fbw_b200::host_threads() : 0;
    // the stages every schedule below runs for a group of sequences or a time chunk
    const int kStages = host_patch ? (kDoGather | kDoSweep | kDoPost) : kDoAll;

    // frames at or past seq_len keep sums = 0 (fbw_op.cu:120-124)
    CUDA_OK(cudaMemsetAsync(sums, 0, sizeof(float) * (size_t)(s.T * s.B), st));

    // Large calls run as a pipeline over time chunks: both sweeps advance `chunk_steps` frames per
    // chunk from the two ends of every sequence.  The gather of the scores a chunk needs runs one
    // chunk ahead on a second stream, and once the sweeps have crossed, the tiles whose alpha and
    // beta are both known are scored, normalised and written out on a third stream while the sweeps
    // go on.  The sweeps are arithmetic-bound, the gather and the output pass memory-bound, so they
    // overlap well; only the first gather chunk and the last output chunk are exposed.
    // Batches whose sequences differ a lot in size (lattices) run instead as size groups: rank
    // ranges of the cost order, each launched with its own thread count and shared-memory size on
    // its own stream, so that small automata do not inherit the footprint of the largest one and
    // several of their CTAs share an SM.
    // Scores in host memory (read over the bus by the gather) make the gather the longest stage by
    // far; the time-chunk pipeline, which keeps it running back to back, is then the better schedule
    // (36.0 against 38.1 ms per call on the triphone workload).  Lattice-like batches keep their
    // groups, which they need for their launch shapes.
    bool host_scores = false;
    {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, am) == cudaSuccess) {
            host_scores = attr.type == cudaMemoryTypeHost;
        } else {
            (void)cudaGetLastError();  // an unregistered pointer is not an error here
        }
        if (cudaPointerGetAttributes(&attr, out) == cudaSuccess) {
            a.out_plain = attr.type == cudaMemoryTypeHost ? 1 : 0;
        } else {
            (void)cudaGetLastError();
        }
        if (host_patch && !a.out_plain) return FBW_B200_BAD_ARGUMENT;
    }
    if (host_help && host_scores) {
        // Scores in host memory: reading the sectors the automata need over the bus takes 37 ms on the
        // triphone workload (32-byte read requests), and nothing else of the call can start before.  The
        // host threads pick them out of the tensor instead (a cache line per class, 13 ms) and one copy
        // takes the 92 MB to the device; k_gather then only builds the tiled copy.
        static int conf = -1;
        if (conf < 0) { const char* e = getenv("FBW_B200_HOST_GATHER"); conf = e ? atoi(e) : 1; }
        if (conf) {
            CUDA_OK(cudaEventSynchronize(host_pool->host_ready));
            host_rows.am = am;
            float* G = reinterpret_cast<float*>(static_cast<char*>(host_work) + H.G);
            if (!fbw_b200::host_gather(host_rows, G, host_nthreads)) return FBW_B200_BAD_ARGUMENT;
            CUDA_OK(cudaMemcpyAsync(a.Gf, G, 4 * (size_t)s.frame_floats, cudaMemcpyHostToDevice, st));
            a.gathered_by_host = 1;
            host_scores = false;  // from here on the call is one whose scores are on the device
        }
    }
    int G = ev ? 1 : choose_groups(s);
    if (G > 1 && host_scores && !(s.max_edges >= 2048 && (double)s.max_edges * (double)s.B >= 1.8 * (double)s.E)) G = 1;
    if (host_patch) G = 1;  // the host's row order follows the time chunks
    i64 ms, me, md;
    plan_maxima(s, ms, me, md);
    // Output in two steps: four groups, most expensive first.  Large calls that can write their output
    // that way run as groups whatever their batch size: with the background written during the sweeps
    // the group schedule beats the time-chunk pipeline also for few sequences (triphone, ms per call,
    // chunks against groups: 8 sequences 1.35 / 1.28, 16: 1.44 / 1.39, 32: 1.79 / 1.70, 48: 2.21 / 1.97;
    // BPE-CTC 32 sequences 0.68 / 0.61).
    const bool groups_forced = getenv("FBW_B200_NUM_GROUPS") != nullptr;
    const bool can_two_step = !ev && fused != 2 && !a.out_plain && (((uintptr_t)out & 31) == 0) &&
                              output_in_two_steps(s, ms, me, md);
    if (can_two_step && G == 1 && !groups_forced && !host_scores && !host_patch && s.B >= 4 &&
        (double)s.T * (double)s.B * (double)s.F >= 1.0e8) {
        G = 4;
    }
    const bool two_step = G > 1 && can_two_step;
    if (two_step && G == 8 && !groups_forced) G = 4;
    const int C = (ev || G > 1) ? 1 : choose_chunks(s);
    // every launch shape is checked before anything is enqueued, so that a call that cannot run
    // fails before it has forked onto the auxiliary streams
    if (s.max_len > 0) {
        if (!sweep_shape(ms, me, md).found) return FBW_B200_TOO_LARGE;
    }
    StreamPool* pool = (C > 1 || G > 1) ? stream_pool() : nullptr;
    // Once work has been forked onto auxiliary streams they are joined back into the caller's
    // stream whatever happens: the caller may release the buffers in stream order after an error.
    int rc_forked = FBW_B200_OK;
    if (G > 1 && pool) {
        std::unique_lock<std::mutex> lock(pool->mu);
        const int per = FBW_B200_GROUPS / G;  // base groups merged into one launch group
        // the cheapest group goes first: its sweeps end first and its output stages start while the
        // expensive groups are still sweeping (FBW_B200_GROUP_ORDER=0: most expensive first)
        static int reverse = -1;
        if (reverse < 0) { const char* e = getenv("FBW_B200_GROUP_ORDER"); reverse = e ? atoi(e) : 1; }
        // Clusters for the groups of the largest automata, most expensive group first, while the
        // call's sweep CTAs stay below 1.65 per SM (the CTAs of short sequences leave early;
        // measured on 64 lattice sequences: 24.6 ms without clusters, 18.6 ms filling the idle SMs
        // only, 15.0 ms with a bound of 1.5, 14.4 ms with 1.65, 14.6 ms with 1.8).
        int group_cs[FBW_B200_GROUPS];
        bool clustered = false;
        {
            static double oversub = -1.0;
            if (oversub < 0) { const char* e = getenv("FBW_B200_CLUSTER_OVERSUB"); oversub = e ? atof(e) : 0.65; }
            int spare = (int)(sm_count() * (1.0 + oversub)) - 2 * (int)s.B;
            // up to four sweep CTAs per SM the most expensive sequences still get clusters worth 15 %
            // more CTAs: their sweeps, not the amount of work, end the call (128 lattice sequences:
            // 26.0 -> 17.7 ms; 256: 31.9 -> 30.6 ms; 512 sequences are better off without: 56 -> 59 ms)
            static double share = -1.0;
            if (share < 0) { const char* e = getenv("FBW_B200_CLUSTER_SHARE"); share = e ? atof(e) : 0.15; }
            if (2 * s.B <= 4 * (i64)sm_count() && spare < (int)(share * 2 * (double)s.B)) {
                spare = (int)(share * 2 * (double)s.B);
            }
            for (int g = 0; g < G; g++) {
                const int r0 = (int)(((i64)(g * per) * s.B) / FBW_B200_GROUPS);
                const int r1 = (int)(((i64)((g + 1) * per) * s.B) / FBW_B200_GROUPS);
                i64 gs_ = 0;
                for (int q = g * per; q < (g + 1) * per; q++) gs_ = s.group_max_states[q] > gs_ ? s.group_max_states[q] : gs_;
                group_cs[g] = sweep_cluster_size(gs_, 2 * (r1 - r0), &spare);
                clustered = clustered || group_cs[g] > 1;
            }
        }
        // with clusters the long sequences are the critical path: they start first
        const bool cheapest_first = reverse && !clustered && !two_step;
        struct GroupRun { int r0, r1, cs; i64 ms, me, md; cudaStream_t st; } runs[FBW_B200_GROUPS];
        int nruns = 0;
        for (int gi = 0; gi < G; gi++) {
            const int g = cheapest_first ? G - 1 - gi : gi;
            GroupRun r;
            r.r0 = (int)(((i64)(g * per) * s.B) / FBW_B200_GROUPS);
            r.r1 = (int)(((i64)((g + 1) * per) * s.B) / FBW_B200_GROUPS);
            if (r.r1 <= r.r0) continue;
            r.ms = r.me = r.md = 0;
            for (int q = g * per; q < (g + 1) * per; q++) {
                r.ms = s.group_max_states[q] > r.ms ? s.group_max_states[q] : r.ms;
                r.me = s.group_max_edges[q] > r.me ? s.group_max_edges[q] : r.me;
                r.md = s.group_max_slots[q] > r.md ? s.group_max_slots[q] : r.md;
            }
            r.cs = group_cs[g];
            r.st = nruns == 0 ? st : pool->aux[nruns];
            runs[nruns++] = r;
        }
        unsigned long long* next_row = reinterpret_cast<unsigned long long*>(at<float>(work, R.next_row));
        if (two_step && cudaMemsetAsync(next_row, 0, sizeof(*next_row) * FBW_B200_GROUPS, st) != cudaSuccess) {
            return FBW_B200_CUDA_ERROR;
        }
        CUDA_OK(cudaEventRecord(pool->fork, st));
        // with the output in two steps the SMs without a sweep CTA get CTAs that only write background
        const int idle_sms = sm_count() - 2 * (int)s.B;
        for (int i = 0; i < nruns; i++) {
            const GroupRun& r = runs[i];
            if (i > 0 && cudaStreamWaitEvent(r.st, pool->fork, 0) != cudaSuccess) {
                rc_forked = FBW_B200_CUDA_ERROR;
                break;
            }
            RunArgs ag = a;
            if (two_step) {
                ag.next_row  = next_row + i;
                ag.fill_ctas = idle_sms > 0 ? (idle_sms + i) / nruns : 0;
                // One filler warp per SM keeps the copy engine busier with few large stores (triphone,
                // 64 sequences: 2.27 ms per call with 8 KB or 4 KB pieces, 2.40 with 2 KB); several sweep
                // CTAs, and filler warps, per SM do better with many small ones (BPE-CTC, 256 sequences:
                // 1.29 ms with 2 KB pieces, 1.34 with 8 KB).
                ag.fill_piece = 2 * s.B > (i64)sm_count() ? 512 : kFillFloats;
            }
            int rc = launch_group(ag, r.r0, r.r1, r.ms, r.me, r.md, s, r.st, nullptr,
                                  two_step ? (kDoGather | kDoSweep | kDoPost | kDoPatch) : kStages, r.cs);
            if (i > 0 && (cudaEventRecord(pool->join[i], r.st) != cudaSuccess ||
                          cudaStreamWaitEvent(st, pool->join[i], 0) != cudaSuccess)) {
                rc = rc != FBW_B200_OK ? rc : FBW_B200_CUDA_ERROR;
            }
            if (rc != FBW_B200_OK) {
                rc_forked = rc;
                break;
            }
        }
    } else if (C > 1 && pool) {
        std::unique_lock<std::mutex> lock(pool->mu);
        a.chunk_steps = (int)(((s.max_len + C - 1) / C + kTile - 1) / kTile * kTile);
        const i64 J = a.chunk_steps;
        // chunks that can have work: scores are first needed before the sweeps cross (the middle
        // of the longest sequence); tiles are complete only after the sweeps of the shortest
        // sequence have crossed
        const int last_gather  = (int)((s.max_len / 2 + kTile) / J);
        const int first_finish = (int)((s.min_len / 2 - kTile > 0 ? s.min_len / 2 - kTile : 0) / J);
        cudaStream_t gs = pool->aux[0];
        CUDA_OK(cudaEventRecord(pool->fork, st));
        auto ok = [&](cudaError_t e) {
            if (e != cudaSuccess && rc_forked == FBW_B200_OK) rc_forked = FBW_B200_CUDA_ERROR;
            return rc_forked == FBW_B200_OK;
        };
        int spare = sm_count() - 2 * (int)s.B;
        const int cs_all = sweep_cluster_size(ms, 2 * (int)s.B, &spare);
        auto stage = [&](int c, cudaStream_t on, int what) {
            a.c_lo = c;
            a.c_hi = c + 1;
            const int rc = launch_group(a, 0, (int)s.B, ms, me, md, s, on, nullptr, what, cs_all);
            if (rc != FBW_B200_OK && rc_forked == FBW_B200_OK) rc_forked = rc;
            return rc_forked == FBW_B200_OK;
        };
        bool go = ok(cudaStreamWaitEvent(gs, pool->fork, 0));
        for (int i = 1; i <= kPostStreams && go; i++) go = ok(cudaStreamWaitEvent(pool->aux[i], pool->fork, 0));
        // Enqueue stage by stage, not chunk by chunk: every gather first, then every sweep chunk,
        // then the output stages.  The streams are independent queues, so the GPU sees the same
        // dependencies, but the sweep chunks (the critical path) are all queued before the host
        // spends time on the many small launches of the output stages.
        for (int c = 0; c < C && c <= last_gather && go; c++) {
            go = stage(c, gs, kDoGather) && ok(cudaEventRecord(pool->gathered[c], gs));
        }
        for (int c = 0; c < C && go; c++) {
            if (c <= last_gather) go = ok(cudaStreamWaitEvent(st, pool->gathered[c], 0));
            go = go && stage(c, st, kDoSweep);
            if (go && (c == 0 || c >= first_finish)) go = ok(cudaEventRecord(pool->swept[c], st));
        }
        // the output stages of successive chunks go to different streams: each stage is a chain
        // of latency-bound kernels, several chunks' chains have to be in flight at once
        bool copied_all = false;
        for (int c = 0; c < C && go; c++) {
            if (!(c == 0 || c >= first_finish)) continue;
            cudaStream_t ps = pool->aux[1 + c % kPostStreams];
            go = ok(cudaStreamWaitEvent(ps, pool->swept[c], 0));
            // (tiles past a sequence's end go with chunk 0: nothing to do for them in host_patch mode)
            if (c >= first_finish) go = go && stage(c, ps, host_patch ? kDoPost : (kDoPost | kDoExpand));
            else if (!host_patch) go = go && stage(c, ps, kDoExpand);
            if (host_patch && c >= first_finish) go = go && ok(cudaEventRecord(host_pool->host_done[c], ps));
            if (go && out_host) {
                // The frames of a 32-frame tile are complete for EVERY sequence once the output
                // stages of the chunk in which the longest sequence finishes that tile have run (a
                // shorter sequence finishes a tile no later; tiles past the longest sequence are
                // padding, written with chunk 0).  Complete tiles are contiguous in the (T,B,F)
                // output, so they go to the host copy while the later chunks are still computed.
                go = ok(cudaEventRecord(pool->expanded[c], ps)) &&
                     ok(cudaStreamWaitEvent(pool->copy, pool->expanded[c], 0));
                const int ntT = (int)((s.T + kTile - 1) / kTile);
                auto tile_chunk = [&](int k) -> int {
                    const int Te = (int)s.max_len;
                    if (k * kTile >= Te) return 0;
                    const int last = (k * kTile + kTile - 1 < Te - 1) ? k * kTile + kTile - 1 : Te - 1;
                    const int a1 = last / (int)J, a2 = (Te - 1 - k * kTile) / (int)J;
                    int dc = a1 > a2 ? a1 : a2;
                    if (dc > 0 && dc < first_finish) dc = first_finish;  // no output stages ran in between
                    return dc;
                };
                for (int k = 0; k < ntT && go;) {
                    if (tile_chunk(k) != c) { k++; continue; }
                    int k1 = k;
                    while (k1 < ntT && tile_chunk(k1) == c) k1++;
                    const i64 f0 = (i64)k * kTile, f1 = (i64)k1 * kTile < s.T ? (i64)k1 * kTile : s.T;
                    const size_t off = (size_t)f0 * (size_t)s.B * (size_t)s.F;
                    go = ok(cudaMemcpyAsync(out_host + off, out + off, (size_t)(f1 - f0) * s.B * s.F * sizeof(float),
                                            cudaMemcpyDeviceToHost, pool->copy));
                    k = k1;
                }
                copied_all = true;
            }
        }
        if (out_host && copied_all) {
            if (cudaEventRecord(pool->copied, pool->copy) != cudaSuccess ||
                cudaStreamWaitEvent(st, pool->copied, 0) != cudaSuccess) {
                if (rc_forked == FBW_B200_OK) rc_forked = FBW_B200_CUDA_ERROR;
            }
            out_host = nullptr;  // done piecewise
        }
        host_first_chunk = first_finish;
        host_chunks = C;
        host_rows.chunk_steps = a.chunk_steps;
        host_rows.first_chunk = first_finish;
        // join: the gather stream and the output streams back into the caller's stream
        for (int i = 0; i <= kPostStreams; i++) {
            if (cudaEventRecord(pool->join[i], pool->aux[i]) != cudaSuccess ||
                cudaStreamWaitEvent(st, pool->join[i], 0) != cudaSuccess) {
                if (rc_forked == FBW_B200_OK) rc_forked = FBW_B200_CUDA_ERROR;
            }
        }
    } else {
        int spare = sm_count() - 2 * (int)s.B;
        int rc = launch_group(a, 0, (int)s.B, ms, me, md, s, st, ev, kStages,
                              sweep_cluster_size(ms, 2 * (int)s.B, &spare));
        if (rc != FBW_B200_OK) return rc;
    }
    if (rc_forked != FBW_B200_OK) return rc_forked;
    if (host_patch) {
        // The device work is enqueued; this thread now writes the rows.  Those past the sequences'
        // ends need no posteriors; the others follow chunk by chunk as the posterior stages finish
        // (a call without time chunks has one chunk, complete when everything on `st` so far is).
        if (host_chunks == 0) {
            CUDA_OK(cudaEventRecord(host_pool->host_done[0], st));
            host_chunks = 1;
        }
        CUDA_OK(cudaEventSynchronize(host_pool->host_ready));
        const bool dbg = getenv("FBW_B200_HOST_DEBUG") != nullptr;
        auto now_ms = []() { timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts); return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6; };
        const double t_start = now_ms();
        bool rows_ok = fbw_b200::host_compose(host_rows, -1, host_nthreads);
        if (dbg) fprintf(stderr, "host: padding rows done at %.1f ms\n", now_ms() - t_start);
        for (int c = host_first_chunk; c < host_chunks; c++) {
            CUDA_OK(cudaEventSynchronize(host_pool->host_done[c]));
            const double t_ready = now_ms();
            rows_ok = fbw_b200::host_compose(host_rows, c, host_nthreads) && rows_ok;
            if (dbg) fprintf(stderr, "host: chunk %d ready at %.1f ms, written at %.1f ms\n", c, t_ready - t_start, now_ms() - t_start);
        }
        if (!rows_ok) return FBW_B200_BAD_ARGUMENT;
    }
    if (out_host) {  // schedules without time chunks: one copy behind everything
        CUDA_OK(cudaMemcpyAsync(out_host, out, (size_t)s.T * s.B * s.F * sizeof(float), cudaMemcpyDeviceToHost, st));
    }
    if (ev) CUDA_OK(cudaEventRecord(ev[4], st));
    if (loss2) {
        k_loss<<<1, 1024, 0, st>>>(sums, s.T, s.B, loss2);
        COUNT_LAUNCH(1);
    }
    if (ev) CUDA_OK(cudaEventRecord(ev[5], st));
    CUDA_OK(cudaGetLastError());
    return FBW_B200_OK;
}

int fbw_b200_run(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                 float* sums, float* loss2, void* work, size_t work_bytes,
                 fbw_b200_stream_t stream) {
    return run_impl(plan, summary, am, out, sums, loss2, work, work_bytes, stream, nullptr);
}

int fbw_b200_run_fused(const void* plan, const fbw_b200_summary* summary, const float* log_probs,
                       float* grad, float* sums, float* loss2, void* work, size_t work_bytes,
                       fbw_b200_stream_t stream) {
    return run_impl(plan, summary, log_probs, grad, sums, loss2, work, work_bytes, stream, nullptr, 1);
}

int fbw_b200_run_for_export(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                            float* sums, float* loss2, void* work, size_t work_bytes,
                            fbw_b200_stream_t stream) {
    return run_impl(plan, summary, am, out, sums, loss2, work, work_bytes, stream, nullptr, 0, 1);
}

int fbw_b200_run_host_out(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                          float* out_host, float* sums, float* loss2, void* work, size_t work_bytes,
                          fbw_b200_stream_t stream) {
    if (!out_host) return FBW_B200_BAD_ARGUMENT;
    return run_impl(plan, summary, am, out, sums, loss2, work, work_bytes, stream, nullptr, 0, 0, out_host);
}

size_t fbw_b200_run_with_host_bytes(const fbw_b200_summary* summary) {
    if (!summary) return 0;
    return host_layout(*summary).total;
}

int fbw_b200_run_with_host(const void* plan, const fbw_b200_summary* summary, const float* am, float* out,
                           float* sums, float* loss2, void* work, size_t work_bytes, void* host_work,
                           size_t host_work_bytes, fbw_b200_stream_t stream) {
    if (!summary || !out || !am) return FBW_B200_BAD_ARGUMENT;
    if (!host_work || ((uintptr_t)host_work & 255) != 0) return FBW_B200_BAD_ARGUMENT;
    if (host_work_bytes < host_layout(*summary).total) return FBW_B200_WORKSPACE;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host_work) != cudaSuccess || attr.type != cudaMemoryTypeHost) {
        (void)cudaGetLastError();
        return FBW_B200_BAD_ARGUMENT;  // has to be pinned: the device reads and writes it
    }
    bool out_on_host = false;
    if (cudaPointerGetAttributes(&attr, out) == cudaSuccess) {
        out_on_host = attr.type == cudaMemoryTypeHost;
    } else {
        (void)cudaGetLastError();
    }
    i64 ms, me, md;
    plan_maxima(*summary, ms, me, md);
    static int conf = -1;  // FBW_B200_HOST_ROWS=0: always let the device's output pass write the rows
    if (conf < 0) { const char* e = getenv("FBW_B200_HOST_ROWS"); conf = e ? atoi(e) : 1; }
    const bool rows_by_host = conf && out_on_host && md * 16 <= summary->F;
    return run_impl(plan, summary, am, out, sums, loss2, work, work_bytes, stream, nullptr, 0, 0, nullptr, host_work,
                    rows_by_host);
}

int fbw_b200_run_phases(const void* plan, const fbw_b200_summary* summary, const float* am,
                        float* out, float* sums, float* loss2, void* work, size_t work_bytes,
                        fbw_b200_stream_t stream, float* phase_ms) {
    if (!phase_ms) return FBW_B200_BAD_ARGUMENT;
    cudaEvent_t ev[FBW_B200_NUM_PHASES + 1];
    for (int i = 0; i <= FBW_B200_NUM_PHASES; i++) CUDA_OK(cudaEventCreate(&ev[i]));
    int rc = run_impl(plan, summary, am, out, sums, loss2, work, work_bytes, stream, ev);
    if (rc == FBW_B200_OK) {
        if (cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
            rc = FBW_B200_CUDA_ERROR;
        }
    }
    for (int i = 0; i < FBW_B200_NUM_PHASES; i++) {
        phase_ms[i] = 0.f;
        if (rc == FBW_B200_OK) cudaEventElapsedTime(&phase_ms[i], ev[i], ev[i + 1]);
    }
    for (int i = 0; i <= FBW_B200_NUM_PHASES; i++) cudaEventDestroy(ev[i]);
    return rc;
}

int64_t fbw_b200_launch_count(void) { return (int64_t)g_launches.load(); }

// ---------------------------------------------------------------------------------------------
// The whole op without any caller-provided or allocated scratch
// ---------------------------------------------------------------------------------------------
// Some hosts of this library may not allocate device memory while they run: an inference server
// whose memory pool is sized and frozen at start-up, or a component that is handed input and output
// buffers by a framework and has no allocator of its own to ask for a plan and a work buffer.  For
// them the plan and the run scratch live in one fixed array inside the library image.  Every GPU
// that loads the library carries the array until the process exits, so it is kept modest: 64 MiB,
// enough for the small and medium workloads (a 32-sequence, 500-frame monophone batch needs about
// 45 MiB), not for the 1 GB of scratch of the large ones.
constexpr size_t kNoAllocBytes = (size_t)64 << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

namespace {
// In host code `g_noalloc_scratch` names a host-side shadow of the device array, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
std::mutex g_noalloc_mu;
void*      g_noalloc_ptr[kMaxDevices]  = {nullptr};
bool       g_noalloc_init[kMaxDevices] = {false};

int noalloc_base(void** base) {
    int dev = 0;
    CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return FBW_B200_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_init[dev]) {
        void* ptr = nullptr;
        CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        if (!ptr) return FBW_B200_CUDA_ERROR;
        g_noalloc_ptr[dev]  = ptr;
        g_noalloc_init[dev] = true;
    }
    *base = g_noalloc_ptr[dev];
    return FBW_B200_OK;
}
}  // namespace

size_t fbw_b200_noalloc_capacity(void) { return kNoAllocBytes; }

int fbw_b200_fbw_noalloc(const float* am, const int32_t* edges, const float* weights,
                         const int32_t* start_end, const int32_t* seq_lens, int64_t T, int64_t B,
                         int64_t F, int64_t E, int64_t S, float* out, float* sums, float* loss2,
                         fbw_b200_stream_t stream) {
    if (!am || !out || !sums) return FBW_B200_BAD_ARGUMENT;
    if (T <= 0 || B <= 0 || F <= 0 || S <= 0 || E < 0) return FBW_B200_BAD_ARGUMENT;
    if (((uintptr_t)out & 15) != 0) return FBW_B200_BAD_ARGUMENT;
    // a fixed cap on the size of the score tensor: this entry runs every stage once, one after
    // another on the caller's stream, which suits small and medium calls only
    if ((double)T * (double)B * (double)F >= 1.0e8) return FBW_B200_TOO_LARGE;
    // the plan at the front of the array, the run scratch behind it; what can be told from the
    // arguments alone is checked before anything runs
    const size_t plan_bytes = (plan_layout(B, E, S).total + 255) & ~(size_t)255;
    if (plan_bytes > kNoAllocBytes) return FBW_B200_TOO_LARGE;
    void* base = nullptr;
    int rc = noalloc_base(&base);  // first call on a device: looks the array's address up
    if (rc != FBW_B200_OK) return rc;
    void* plan = base;
    rc = prepare_impl(edges, weights, start_end, seq_lens, T, B, F, E, S, plan, plan_bytes, stream, true);
    if (rc != FBW_B200_OK) return rc;
    fbw_b200_summary sum;
    rc = fbw_b200_plan_summary(plan, &sum, stream);  // synchronises the stream
    if (rc == FBW_B200_RETRY_GENERAL) {
        rc = prepare_impl(edges, weights, start_end, seq_lens, T, B, F, E, S, plan, plan_bytes, stream,
                          false);
        if (rc != FBW_B200_OK) return rc;
        rc = fbw_b200_plan_summary(plan, &sum, stream);
    }
    if (rc != FBW_B200_OK) return rc;
    // the size of the run scratch is known only now; the plan kernels have run on the array, the
    // caller's outputs are untouched
    const RunLayout R = run_layout(sum);
    if (plan_bytes + R.total > kNoAllocBytes) return FBW_B200_TOO_LARGE;
    void* work = static_cast<unsigned char*>(base) + plan_bytes;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    RunArgs a = fbw_args(plan, sum, work, R, am, out, sums, loss2, 0);

    // The array keeps whatever the previous call left in it.  The plan builder clears its own
    // counters; of the run, only the sums must start at zero (the kernels write every other word
    // they later read).
    CUDA_OK(cudaMemsetAsync(sums, 0, sizeof(float) * (size_t)(sum.T * sum.B), st));
    i64 ms, me, md;
    plan_maxima(sum, ms, me, md);
    int spare = sm_count() - 2 * (int)sum.B;
    rc = launch_group(a, 0, (int)sum.B, ms, me, md, sum, st, nullptr, kDoAll,   // one stream, one chunk
                      sweep_cluster_size(ms, 2 * (int)sum.B, &spare));
    if (rc != FBW_B200_OK) return rc;
    if (loss2) {
        k_loss<<<1, 1024, 0, st>>>(sums, sum.T, sum.B, loss2);
        COUNT_LAUNCH(1);
    }
    CUDA_OK(cudaGetLastError());
    return FBW_B200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// debug export: the forward state scores of the last run, dense and indexed by global state id
// ---------------------------------------------------------------------------------------------
namespace {

// thread per (frame, global state); consecutive threads walk the states of one frame, so the
// (T,S) destination is written coalesced
__global__ void k_export_alpha(const float* __restrict__ A, const int* __restrict__ state_key,
                               const int* __restrict__ packed_of, const int* __restrict__ state_off,
                               const int* __restrict__ seq_T, const int* __restrict__ start_l,
                               const i64* __restrict__ ta_off, i64 T, i64 S, float* __restrict__ dst) {
    const i64 n = T * S;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
        const int t = (int)(i / S);
        const int g = (int)(i - (i64)t * S);
        const int q = state_key[g];
        float v = CUDART_INF_F;
        if (q >= 0) {
            const int s0 = state_off[q], Sb = state_off[q + 1] - s0;
            const int l  = packed_of[g] - s0;
            const int Te = seq_T[q];
            if (t < Te) {
                v = A[ta_off[q] + ((i64)(t >> 5) * Sb + l) * kTile + (t & 31)];
            } else if (t == 0) {
                v = l == start_l[q] ? 0.f : CUDART_INF_F;  // the initial vector (fbw_op.cu:297-302)
            }
        }
        dst[i] = v;
    }
}

}  // namespace

extern "C" int fbw_b200_export_alpha(const void* plan, const fbw_b200_summary* summary,
                                     const void* work, size_t work_bytes, float* alpha,
                                     fbw_b200_stream_t stream) {
    if (!plan || !summary || !work || !alpha) return FBW_B200_BAD_ARGUMENT;
    if (summary->error) return FBW_B200_BAD_AUTOMATON;
    const fbw_b200_summary& s = *summary;
    const RunLayout R = run_layout(s);
    if (work_bytes < R.total) return FBW_B200_WORKSPACE;
    const PlanLayout L = plan_layout(s.B, s.E, s.S);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const i64 n = s.T * s.S;
    i64 blocks = (n + 255) / 256;
    const i64 cap = (i64)sm_count() * 16;
    k_export_alpha<<<(int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap), 256, 0, st>>>(
        at<float>(work, R.A), at<int>(plan, L.state_key),
        at<int>(plan, L.packed_of), at<int>(plan, L.state_off),
        at<int>(plan, L.seq_T), at<int>(plan, L.start_l),
        at<i64>(plan, L.ta_off), s.T, s.S, alpha);
    COUNT_LAUNCH(1);
    CUDA_OK(cudaGetLastError());
    return FBW_B200_OK;
}

#include "viterbi_b200.inc"
#include "topology_b200.inc"
