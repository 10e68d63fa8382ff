/* TEST INFRASTRUCTURE ONLY -- CPU oracle for the best-path (Viterbi) alignment.
 *
 * A plain C restatement of what the reference's launcher  fast_viterbi_cuda()
 * (i6_native_ops/fast_viterbi/core.cu:174-275) computes, written from its behaviour:
 *
 *   - a (T+1, S) table of (value, edge) pairs, all (-inf, -1), with value 0 at every start state
 *     of frame 0                                                  (core.cu:50-77, 217-220);
 *   - for t = 0..T-1 every edge whose sequence still has frames (t < seq_len) proposes
 *     (table[t][from].value + weight) + am[t, seq, emission]  for table[t+1][to]; the largest
 *     value wins and, among equal values, the smallest edge index; a proposal of -inf never
 *     replaces the initial (-inf, -1)                              (core.cu:23-48, 79-121);
 *   - score[b] = table[seq_len[b]][end[b]].value                  (core.cu:123-142);
 *   - back-trace from the end state, t = T-1..0: for t < seq_len the recorded edge of
 *     table[t+1][cur] gives output[t,b] = its emission and cur = its source; a missing edge
 *     gives output 0 and leaves cur where it is; frames t >= seq_len give 0   (core.cu:144-172).
 *
 * Scores are POSITIVE log probabilities here (larger is better), unlike the fbw op.
 * The CUDA reference resolves its races with a compare-and-swap loop whose outcome does not
 * depend on thread order (as long as no value is NaN), so this sequential form is exact:
 * alignment and scores must agree bit for bit.
 *
 * A seq_len outside [0, T] makes the reference read past its table; here such a sequence is
 * treated as empty (no frames, score -inf unless start == end).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

typedef struct {
    int32_t idx;
    float   val;
} cell_t;

/* am (T,B,F) f32; edges (4,E) i32 rows from/to/emission/sequence; weights (E); start_end (2,B);
 * seq_lens (B); alignment (T,B) i32 out; scores (B) f32 out.  Returns 0, or a negative code for
 * an index out of range. */
int viterbi_oracle_f32(const float* am, int64_t T, int64_t B, int64_t F, const int32_t* edges,
                       int64_t E, const float* weights, const int32_t* start_end,
                       const int32_t* seq_lens, int64_t S, int32_t* alignment, float* scores) {
    const int32_t *from = edges, *to = edges + E, *emis = edges + 2 * E, *seq = edges + 3 * E;
    for (int64_t e = 0; e < E; e++) {
        if (from[e] < 0 || from[e] >= S || to[e] < 0 || to[e] >= S) return -1;
        if (emis[e] < 0 || emis[e] >= F) return -2;
        if (seq[e] < 0 || seq[e] >= B) return -3;
    }
    for (int64_t b = 0; b < 2 * B; b++) {
        if (start_end[b] < 0 || start_end[b] >= S) return -4;
    }
    cell_t* table = (cell_t*)malloc(sizeof(cell_t) * (size_t)((T + 1) * (S > 0 ? S : 1)));
    int32_t* len  = (int32_t*)malloc(sizeof(int32_t) * (size_t)(B > 0 ? B : 1));
    if (!table || !len) {
        free(table);
        free(len);
        return -5;
    }
    for (int64_t b = 0; b < B; b++) len[b] = (seq_lens[b] >= 0 && seq_lens[b] <= T) ? seq_lens[b] : 0;
    for (int64_t i = 0; i < (T + 1) * S; i++) {
        table[i].idx = -1;
        table[i].val = -INFINITY;
    }
    for (int64_t b = 0; b < B; b++) table[start_end[b]].val = 0.f;

    for (int64_t t = 0; t < T; t++) {
        const cell_t* prev = table + t * S;
        cell_t*       next = table + (t + 1) * S;
        for (int64_t e = 0; e < E; e++) { /* ascending edge index: the first maximum is kept */
            if (t >= len[seq[e]]) continue;
            const float v = (prev[from[e]].val + weights[e]) + am[(t * B + seq[e]) * F + emis[e]];
            cell_t*     c = &next[to[e]];
            if (v > c->val) {
                c->val = v;
                c->idx = (int32_t)e;
            }
        }
    }
    for (int64_t b = 0; b < B; b++) {
        scores[b] = table[(int64_t)len[b] * S + start_end[B + b]].val;
        int32_t cur = start_end[B + b];
        for (int64_t t = T - 1; t >= 0; t--) {
            int32_t o = 0;
            if (t < len[b]) {
                const int32_t e = table[(t + 1) * S + cur].idx;
                if (e >= 0) {
                    cur = from[e];
                    o   = emis[e];
                }
            }
            alignment[t * B + b] = o;
        }
    }
    free(table);
    free(len);
    return 0;
}
