// Host side of the result delivery into pinned host memory (host_fill.cpp): CPU threads compose the
// rows of a sparse (T,B,F) result from the class posteriors the device leaves in pinned host memory.
#pragma once
#include <cstddef>
#include <cstdint>

namespace fbw_b200 {

// Number of host threads: the CPUs this process may run on, shared out over the processes of the
// node when LOCAL_WORLD_SIZE says there are several, at most 16; FBW_B200_HOST_THREADS overrides (1..64).
int host_threads();

// What the host needs to know to write row (t, b) of the output: the sequence's length, its classes
// in ascending order and where its posteriors of frame t are.  All pointers are host memory.
struct HostRows {
    int64_t T, B, F;
    const int*     seq_T;      // [B] valid frames of a sequence (0: none)
    const int*     nslot;      // [B] distinct emission classes of a sequence
    const int*     slot_off;   // [B] first entry of the sequence in slot_emis
    const int64_t* gf_off;     // [B] first float of the sequence in P
    const int*     slot_emis;  // classes, ascending per sequence
    const float*   P;          // posteriors [sequence][frame][slot, padded to 4]
    float*         out;        // (T,B,F)
    const float*   am;         // scores, for host_gather (may be null otherwise): (T,B,F), or
    int            batch_major;  // (B,T,F) if set (the Viterbi op's other layout)
    int chunk_steps;           // frames the sweeps advance per time chunk (1 << 30: one chunk)
    int first_chunk;           // first chunk whose posterior stages ran
    int64_t num_slots, p_floats;  // capacity of slot_emis and of P (the indices above are checked against them)
};

// Chunk after which the posteriors of frame t of a sequence of Te frames exist (both sweeps have
// passed its 32-frame tile); -1 for a frame at or past the sequence's end, which has none.
int host_row_chunk(const HostRows& h, int64_t t, int b);

// Writes every row whose host_row_chunk is `chunk`: +inf everywhere, the posteriors at the
// sequence's classes; rows of chunk -1 are all +inf.  Runs on `threads` threads and returns when
// they are done.  Rows are 48 KB or so of streaming stores each; the posteriors are read once.
// Returns false, with the offending rows left unwritten, if an index of the plan arrays points outside
// slot_emis, P or the row (which a plan accepted by fbw_b200_plan_summary never does).
bool host_compose(const HostRows& h, int chunk, int threads);

// The scores the automata refer to, picked out of h.am by `threads` host threads:
// G[gf_off[b] + t * Dp + d] = am[t][b][class d of sequence b] for every valid frame, 0 in the padding
// slots (Dp = slots padded to 4), the layout of the device's frame-major score array.  Returns false
// on an index outside the arrays (see host_compose).
bool host_gather(const HostRows& h, float* G, int threads);

}  // namespace fbw_b200
