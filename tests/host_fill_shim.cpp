// C entry points around csrc/host_fill.cpp for tests/test_host_fill.py (ctypes); test infrastructure only.
#include "host_fill.h"

extern "C" {

int shim_compose(long long T, long long B, long long F, const int* seq_T, const int* nslot, const int* slot_off,
                 const long long* gf_off, const int* slot_emis, long long num_slots, const float* P,
                 long long p_floats, float* out, int chunk_steps, int first_chunk, int chunk, int threads) {
    fbw_b200::HostRows h;
    h.T = T; h.B = B; h.F = F;
    h.seq_T = seq_T; h.nslot = nslot; h.slot_off = slot_off;
    h.gf_off = reinterpret_cast<const int64_t*>(gf_off);
    h.slot_emis = slot_emis; h.P = P; h.out = out; h.am = nullptr; h.batch_major = 0;
    h.chunk_steps = chunk_steps; h.first_chunk = first_chunk; h.num_slots = num_slots; h.p_floats = p_floats;
    return fbw_b200::host_compose(h, chunk, threads) ? 0 : 1;
}

int shim_gather(long long T, long long B, long long F, const int* seq_T, const int* nslot, const int* slot_off,
                const long long* gf_off, const int* slot_emis, long long num_slots, const float* am,
                int batch_major, float* G, long long g_floats, int threads) {
    fbw_b200::HostRows h;
    h.T = T; h.B = B; h.F = F;
    h.seq_T = seq_T; h.nslot = nslot; h.slot_off = slot_off;
    h.gf_off = reinterpret_cast<const int64_t*>(gf_off);
    h.slot_emis = slot_emis; h.P = nullptr; h.out = nullptr; h.am = am; h.batch_major = batch_major;
    h.chunk_steps = 1 << 30; h.first_chunk = 0; h.num_slots = num_slots; h.p_floats = g_floats;
    return fbw_b200::host_gather(h, G, threads) ? 0 : 1;
}

int shim_row_chunk(int Te, long long t, int chunk_steps, int first_chunk) {
    fbw_b200::HostRows h;
    h.T = t + 1; h.B = 1; h.F = 1;
    h.seq_T = &Te;
    h.chunk_steps = chunk_steps; h.first_chunk = first_chunk;
    return fbw_b200::host_row_chunk(h, t, 0);
}

int shim_threads() { return fbw_b200::host_threads(); }

}
