// Host side of calls whose scores or results live in pinned host memory (fbw_b200_run_with_host).
// Result: the (T,B,F) result of a call with few classes per sequence is almost entirely +inf; sending
// it over the bus costs more than the whole computation.  Instead the device leaves the class
// posteriors (2 % of the result) in pinned host memory as it computes them, and the threads here write
// the rows: a row buffer that holds +inf gets the row's posteriors, goes to its place with streaming
// stores, and has the posteriors taken out again.  Scores: the threads pick the entries the automata
// refer to out of the tensor, which the device would otherwise fetch as 32-byte reads over the bus.
// No counterpart in the reference, whose inputs and outputs are device tensors.
#include "host_fill.h"

#include <emmintrin.h>
#include <sched.h>

#include <atomic>
#include <cstdlib>
#include <limits>
#include <thread>
#include <vector>

namespace fbw_b200 {

int host_threads() {
    if (const char* e = std::getenv("FBW_B200_HOST_THREADS")) {
        const int n = std::atoi(e);
        if (n >= 1 && n <= 64) return n;
    }
    int n = 0;
    cpu_set_t set;
    CPU_ZERO(&set);
    if (sched_getaffinity(0, sizeof(set), &set) == 0) n = CPU_COUNT(&set);
    if (n <= 0) n = (int)std::thread::hardware_concurrency();
    if (n <= 0) n = 1;
    // one process per GPU: the processes of a node share its CPUs (torchrun exports their number)
    if (const char* e = std::getenv("LOCAL_WORLD_SIZE")) {
        const int local = std::atoi(e);
        if (local > 1) n = n / local > 2 ? n / local : 2;
    }
    return n > 16 ? 16 : n;
}

int host_row_chunk(const HostRows& h, int64_t t, int b) {
    const int Te = h.seq_T[b];
    if (t >= Te) return -1;
    const int k = (int)(t / 32);
    const int last = k * 32 + 31 < Te - 1 ? k * 32 + 31 : Te - 1;
    const int fwd = last / h.chunk_steps, bwd = (Te - 1 - k * 32) / h.chunk_steps;
    const int c = fwd > bwd ? fwd : bwd;
    return c < h.first_chunk ? h.first_chunk : c;
}

namespace {

// dst[0, n) <- src[0, n), dst and src equally aligned modulo 16 bytes; streaming stores for the body
void copy_out(float* dst, const float* src, int64_t n) {
    int64_t i = 0;
    while (i < n && (reinterpret_cast<uintptr_t>(dst + i) & 15) != 0) { dst[i] = src[i]; i++; }
    for (; i + 16 <= n; i += 16) {
        _mm_stream_ps(dst + i, _mm_load_ps(src + i));
        _mm_stream_ps(dst + i + 4, _mm_load_ps(src + i + 4));
        _mm_stream_ps(dst + i + 8, _mm_load_ps(src + i + 8));
        _mm_stream_ps(dst + i + 12, _mm_load_ps(src + i + 12));
    }
    for (; i + 4 <= n; i += 4) _mm_stream_ps(dst + i, _mm_load_ps(src + i));
    for (; i < n; i++) dst[i] = src[i];
}

void worker(const HostRows* hp, int chunk, std::atomic<int64_t>* next, std::atomic<int>* bad) {
    const HostRows& h = *hp;
    const float inf = std::numeric_limits<float>::infinity();
    // the row buffer, with room to give it the alignment of the destination row
    std::vector<float> store((size_t)h.F + 32, inf);
    float* aligned = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(store.data()) + 63) & ~(uintptr_t)63);
    const int64_t rows = h.T * h.B;
    const int64_t batch = 8;  // rows taken at a time
    for (;;) {
        const int64_t r0 = next->fetch_add(batch);
        if (r0 >= rows) break;
        const int64_t r1 = r0 + batch < rows ? r0 + batch : rows;
        for (int64_t r = r0; r < r1; r++) {
            const int64_t t = r / h.B;
            const int b = (int)(r - t * h.B);
            if (host_row_chunk(h, t, b) != chunk) continue;
            float* dst = h.out + r * h.F;
            float* buf = aligned + ((reinterpret_cast<uintptr_t>(dst) & 63) >> 2);
            const bool valid = chunk >= 0;
            const int Db = valid ? h.nslot[b] : 0;
            const int64_t so = h.slot_off[b], po = h.gf_off[b] + t * (int64_t)((h.nslot[b] + 3) & ~3);
            if (Db < 0 || (Db > 0 && (so < 0 || so + Db > h.num_slots || po < 0 || po + Db > h.p_floats))) {
                bad->store(1);
                continue;
            }
            const int* emis = h.slot_emis + so;
            const float* post = h.P + po;
            bool in_row = true;
            for (int d = 0; d < Db; d++) in_row = in_row && emis[d] >= 0 && emis[d] < h.F;
            if (!in_row) {
                bad->store(1);
                continue;
            }
            for (int d = 0; d < Db; d++) buf[emis[d]] = post[d];
            copy_out(dst, buf, h.F);
            for (int d = 0; d < Db; d++) buf[emis[d]] = inf;
        }
    }
    _mm_sfence();
}

}  // namespace

namespace {

void gather_worker(const HostRows* hp, float* G, std::atomic<int64_t>* next, std::atomic<int>* bad) {
    const HostRows& h = *hp;
    const int64_t rows = h.T * h.B;
    const int64_t batch = 16;
    for (;;) {
        const int64_t r0 = next->fetch_add(batch);
        if (r0 >= rows) break;
        const int64_t r1 = r0 + batch < rows ? r0 + batch : rows;
        for (int64_t r = r0; r < r1; r++) {
            const int64_t t = r / h.B;
            const int b = (int)(r - t * h.B);
            if (t >= h.seq_T[b]) continue;
            const int Db = h.nslot[b], Dp = (Db + 3) & ~3;
            const int64_t so = h.slot_off[b], po = h.gf_off[b] + t * (int64_t)Dp;
            if (Db < 0 || so < 0 || so + Db > h.num_slots || po < 0 || po + Dp > h.p_floats) {
                bad->store(1);
                continue;
            }
            const int* emis = h.slot_emis + so;
            const float* row = h.am + (h.batch_major ? (int64_t)b * h.T + t : r) * h.F;
            float* g = G + po;
            // the reads are the cost (a cache line of the score row per class): ask for them ahead
            for (int d = 0; d < Db && d < 16; d++) _mm_prefetch(reinterpret_cast<const char*>(row + emis[d]), _MM_HINT_NTA);
            for (int d = 0; d < Db; d++) {
                if (d + 16 < Db) _mm_prefetch(reinterpret_cast<const char*>(row + emis[d + 16]), _MM_HINT_NTA);
                const int e = emis[d];
                if (e < 0 || e >= h.F) {
                    bad->store(1);
                    break;
                }
                g[d] = row[e];
            }
            for (int d = Db; d < Dp; d++) g[d] = 0.f;
        }
    }
}

}  // namespace

bool host_gather(const HostRows& h, float* G, int threads) {
    if (threads < 1) threads = 1;
    std::atomic<int64_t> next{0};
    std::atomic<int> bad{0};
    std::vector<std::thread> pool;
    pool.reserve((size_t)threads - 1);
    // (a thread that cannot be started is not an error: the rows are handed out through `next`, and
    // the threads that do run, this one included, take them all)
    for (int i = 1; i < threads; i++) {
        try {
            pool.emplace_back(gather_worker, &h, G, &next, &bad);
        } catch (...) {
            break;
        }
    }
    gather_worker(&h, G, &next, &bad);
    for (auto& th : pool) th.join();
    return bad.load() == 0;
}

bool host_compose(const HostRows& h, int chunk, int threads) {
    if (threads < 1) threads = 1;
    std::atomic<int64_t> next{0};
    std::atomic<int> bad{0};
    std::vector<std::thread> pool;
    pool.reserve((size_t)threads - 1);
    for (int i = 1; i < threads; i++) {
        try {
            pool.emplace_back(worker, &h, chunk, &next, &bad);
        } catch (...) {
            break;  // see host_gather
        }
    }
    worker(&h, chunk, &next, &bad);
    for (auto& th : pool) th.join();
    return bad.load() == 0;
}

}  // namespace fbw_b200
