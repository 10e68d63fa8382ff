// fbw_torch.cpp -- torch extension `fbw_core`: the Python-visible op over the C ABI of
// include/fbw_b200.h.  Mirrors the reference binding i6_native_ops/fbw/fbw_torch.cpp:15-40:
// same module members (`fbw`, `DebugOptions`), same seven positional arguments, same input
// checks (CUDA, contiguous, dtype -> RuntimeError), same two outputs, same text dumps under
// DebugOptions.
//
// Differences that do not change results: scratch comes from torch's caching allocator instead
// of cudaMalloc/cudaFree per call (fbw_op.cu:283-286, 384-389); work is enqueued on torch's current
// stream of the inputs' device under a device guard (the reference uses the legacy default stream
// and the current device, common/returnn_definitions.h:29); sizes are 64-bit.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <atomic>
#include <cmath>
#include <fstream>
#include <limits>
#include <sstream>
#include <vector>

#include "fbw_b200.h"
#include "torch_common.h"

namespace py = pybind11;

namespace fbw_b200 {
// Same fields and defaults as the reference's DebugOptions (i6_native_ops/fbw/DebugOptions.h:4-9).
// Lives in its own namespace and is registered module-local so that this module and the
// reference's can be imported into one process.
struct DebugOptions {
    bool     dump_alignment = false;
    bool     dump_output    = false;
    unsigned dump_every     = 40u;
    float    pruning        = 10.f;
};
}  // namespace fbw_b200
using fbw_b200::DebugOptions;
using namespace fbw_b200::torch_glue;

namespace {

std::vector<torch::Tensor> run_impl(const Prepared& p, const torch::Tensor& am_scores,
                                    bool want_loss, torch::Tensor out = torch::Tensor(),
                                    torch::Tensor sums = torch::Tensor(),
                                    torch::Tensor* work_out = nullptr, bool for_export = false) {
    auto stream = at::cuda::getCurrentCUDAStream();
    const fbw_b200_summary& s = p.summary;
    if (!out.defined()) out = torch::empty_like(am_scores);
    if (!sums.defined()) sums = torch::empty({s.T, s.B}, am_scores.options());
    torch::Tensor loss2;
    if (want_loss) loss2 = torch::empty({2}, am_scores.options());
    size_t wbytes = fbw_b200_run_bytes(&s);
    torch::Tensor work = byte_buffer(wbytes, am_scores.device());
    // a call whose forward scores will be dumped computes them for every state, as the reference does
    auto run = for_export ? fbw_b200_run_for_export : fbw_b200_run;
    check_status(run(p.plan.data_ptr(), &s, am_scores.data_ptr<float>(), out.data_ptr<float>(),
                     sums.data_ptr<float>(), want_loss ? loss2.data_ptr<float>() : nullptr,
                     work.data_ptr(), wbytes, reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
    if (work_out) *work_out = work;
    if (want_loss) return {out, sums, loss2};
    return {out, sums};
}

// The reference's text dumps (fbw_op.cu:155-224), written into the current directory like there.
// alignment.dump.<call>.<seq>: per frame t < seq_len (frame 0 always) the forward state scores of the
// states start..end of the sequence, normalised over those states, one line "t local_state value" for
// every value <= pruning.  target.dump.<call>.<seq>: per frame the output values <= pruning, one line
// "t emission value".  Values are printed by a default-formatted ostream (6 significant digits).
void write_alignment_dump(const torch::Tensor& alpha_dev, const torch::Tensor& start_end_states,
                          const torch::Tensor& seq_lens, float pruning, unsigned call_idx) {
    torch::Tensor alpha = alpha_dev.cpu();
    torch::Tensor se = start_end_states.cpu(), sl = seq_lens.cpu();
    const int64_t T = alpha.size(0), S = alpha.size(1), B = sl.size(0);
    const float*   a    = alpha.data_ptr<float>();
    const int32_t* sep  = se.data_ptr<int32_t>();
    const int32_t* lens = sl.data_ptr<int32_t>();
    for (int64_t b = 0; b < B; b++) {
        std::ostringstream name;
        name << "alignment.dump." << call_idx << '.' << b;
        std::ofstream f(name.str().c_str(), std::ios::out | std::ios::trunc);
        const int64_t first = sep[b], last = sep[B + b];
        const uint32_t len = (uint32_t)lens[b];  // the reference keeps lengths unsigned
        for (int64_t t = 0; t < T && !(t > 0 && (uint64_t)t >= len); t++) {
            const float* row = a + t * S;
            float total = std::numeric_limits<float>::infinity();
            for (int64_t s = first; s <= last; s++) {
                const float d = row[s] - total;
                if (!std::isnan(d)) total = -log1pf(expf(-fabsf(d))) + fminf(total, row[s]);
            }
            for (int64_t s = first; s <= last; s++) {
                const float v = row[s] - total;
                if (v <= pruning) f << t << ' ' << (s - first) << ' ' << v << '\n';
            }
        }
    }
}

void write_output_dump(const torch::Tensor& out_dev, const torch::Tensor& seq_lens, float pruning,
                       unsigned call_idx) {
    torch::Tensor out = out_dev.cpu(), sl = seq_lens.cpu();
    const int64_t T = out.size(0), B = out.size(1), F = out.size(2);
    const float*   o    = out.data_ptr<float>();
    const int32_t* lens = sl.data_ptr<int32_t>();
    for (int64_t b = 0; b < B; b++) {
        std::ostringstream name;
        name << "target.dump." << call_idx << '.' << b;
        std::ofstream f(name.str().c_str(), std::ios::out | std::ios::trunc);
        const uint32_t len = (uint32_t)lens[b];
        for (int64_t t = 0; t < T && !(t > 0 && (uint64_t)t >= len); t++) {
            const float* row = o + (t * B + b) * F;
            for (int64_t e = 0; e < F; e++) {
                if (row[e] <= pruning) f << t << ' ' << e << ' ' << row[e] << '\n';
            }
        }
    }
}

}  // namespace

// The op.  Signature and meaning of the reference's fbw() (fbw_torch.cpp:15-29): am_scores (T,B,F)
// f32 negative log scores, edges (4,E) i32, weights (E) f32, start_end_states (2,B) i32, seq_lens
// (B) i32, num_states -> [out (T,B,F) negative log posteriors, sum_output (T,B)].
std::vector<torch::Tensor> fbw(torch::Tensor& am_scores, torch::Tensor& edges,
                               torch::Tensor& weights, torch::Tensor& start_end_states,
                               torch::Tensor& seq_lens, unsigned num_states,
                               DebugOptions debug_options) {
    check_input(am_scores, torch::kFloat32, "am_scores");
    TORCH_CHECK(am_scores.dim() == 3, "am_scores must have shape (T, B, F)");
    TORCH_CHECK(start_end_states.dim() == 2 && start_end_states.size(1) == am_scores.size(1),
                "start_end_states must have shape (2, B) with B = am_scores.size(1)");
    check_input(edges, torch::kInt32, "edges");
    check_same_device(am_scores, edges);
    c10::cuda::CUDAGuard guard(am_scores.device());
    // the outputs do not depend on the plan: allocate them while the plan is still being built
    torch::Tensor out  = torch::empty_like(am_scores);
    torch::Tensor sums = torch::empty({am_scores.size(0), am_scores.size(1)}, am_scores.options());
    Prepared p = prepare_impl(edges, weights, start_end_states, seq_lens, am_scores.size(0),
                              am_scores.size(2), (int64_t)num_states);
    // dumps every `dump_every`-th call of the process, counted like the reference's static batch_idx
    // (fbw_op.cu:246, 390)
    static std::atomic<unsigned> call_counter{0};
    const unsigned call_idx = call_counter.fetch_add(1);
    const bool dump_now = debug_options.dump_every > 0 && call_idx % debug_options.dump_every == 0;
    torch::Tensor work;
    auto result = run_impl(p, am_scores, false, out, sums, &work, dump_now && debug_options.dump_alignment);
    if (dump_now && debug_options.dump_alignment) {
        auto stream = at::cuda::getCurrentCUDAStream();
        torch::Tensor alpha = torch::empty({p.summary.T, p.summary.S}, am_scores.options());
        check_status(fbw_b200_export_alpha(p.plan.data_ptr(), &p.summary, work.data_ptr(),
                                           (size_t)work.numel(), alpha.data_ptr<float>(),
                                           reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
        write_alignment_dump(alpha, start_end_states, seq_lens, debug_options.pruning, call_idx);
    }
    if (dump_now && debug_options.dump_output) {
        write_output_dump(out, seq_lens, debug_options.pruning, call_idx);
    }
    return result;
}

// The op on scores that live in PINNED HOST memory: am_scores (T,B,F) f32, a pinned CPU tensor, is
// not copied to the device as a whole; the gather kernel reads the scores the automata need (one
// 32-byte sector per distinct (frame, sequence, emission)) straight out of host memory through the
// unified address space, which moves a fraction of the tensor over the bus.  Everything else, and the
// results, are those of fbw().  With `out_pinned` the (T,B,F) result is delivered into that pinned host
// tensor (see the comment inside); sums and loss2 stay on the device.
// No counterpart in the reference, which requires CUDA tensors (fbw_torch.cpp:19-23).
std::vector<torch::Tensor> fbw_host_scores(torch::Tensor& am_scores, torch::Tensor& edges,
                                           torch::Tensor& weights, torch::Tensor& start_end_states,
                                           torch::Tensor& seq_lens, int64_t num_states,
                                           c10::optional<torch::Tensor> out_pinned, bool staged) {
    TORCH_CHECK(!am_scores.is_cuda() && am_scores.is_pinned(),
                "am_scores must be a pinned host tensor (use fbw() for CUDA tensors)");
    TORCH_CHECK(am_scores.is_contiguous() && am_scores.scalar_type() == torch::kFloat32,
                "am_scores must be contiguous float32");
    TORCH_CHECK(am_scores.dim() == 3, "am_scores must have shape (T, B, F)");
    TORCH_CHECK(edges.is_cuda(), "edges must be a CUDA tensor");
    TORCH_CHECK(start_end_states.dim() == 2 && start_end_states.size(1) == am_scores.size(1),
                "start_end_states must have shape (2, B) with B = am_scores.size(1)");
    c10::cuda::CUDAGuard guard(edges.device());
    auto dev_opts = weights.options();  // float32 on the automata's device
    torch::Tensor out, out_dev;
    if (out_pinned.has_value()) {
        // The (T,B,F) result ends up in the caller's pinned host tensor.  staged: the library picks the
        // faster way over the bus -- where the rows are sparse, only the class posteriors are sent and
        // host threads write the rows from them while the device goes on (fbw_b200_run_with_host; the
        // call then returns when the rows are written); else the result is produced in a device buffer
        // and copied out piece by piece while the rest is still being computed.  Not staged: the
        // output pass writes every row straight into host memory.  No device copy of the result is
        // kept in either case.
        out = *out_pinned;
        TORCH_CHECK(!out.is_cuda() && out.is_pinned() && out.is_contiguous() &&
                        out.scalar_type() == torch::kFloat32 && out.sizes() == am_scores.sizes(),
                    "out must be a pinned contiguous float32 host tensor of the shape of am_scores");
    } else {
        out = torch::empty(am_scores.sizes(), dev_opts);
    }
    torch::Tensor sums = torch::empty({am_scores.size(0), am_scores.size(1)}, dev_opts);
    Prepared p = prepare_impl(edges, weights, start_end_states, seq_lens, am_scores.size(0),
                              am_scores.size(2), num_states);
    auto   stream = at::cuda::getCurrentCUDAStream();
    size_t wbytes = fbw_b200_run_bytes(&p.summary);
    torch::Tensor work  = byte_buffer(wbytes, edges.device());
    torch::Tensor loss2 = torch::empty({2}, dev_opts);
    // pinned host memory is addressable from the device under unified addressing
    const bool sparse_rows = p.summary.max_slots * 16 <= p.summary.F;
    // Host threads of the library help where the rows are sparse: they pick the scores the automata
    // need out of the pinned tensor (instead of 32-byte reads over the bus) and, for a result in host
    // memory, write its rows from the posteriors the device sends.  Small calls are not worth the threads.
    const bool with_host = sparse_rows && (double)am_scores.numel() >= 1.0e7 &&
                           (out_pinned.has_value() ? staged : true);
    if (with_host) {
        const size_t hbytes = fbw_b200_run_with_host_bytes(&p.summary);
        torch::Tensor host_work = torch::empty({(int64_t)hbytes}, torch::TensorOptions().dtype(torch::kUInt8).pinned_memory(true));
        check_status(fbw_b200_run_with_host(p.plan.data_ptr(), &p.summary, am_scores.data_ptr<float>(),
                                            out.data_ptr<float>(), sums.data_ptr<float>(), loss2.data_ptr<float>(),
                                            work.data_ptr(), wbytes, host_work.data_ptr(), hbytes,
                                            reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
        return {out, sums, loss2};
    }
    if (out_pinned.has_value() && staged) out_dev = torch::empty(am_scores.sizes(), dev_opts);
    if (out_dev.defined()) {
        check_status(fbw_b200_run_host_out(p.plan.data_ptr(), &p.summary, am_scores.data_ptr<float>(),
                                           out_dev.data_ptr<float>(), out.data_ptr<float>(),
                                           sums.data_ptr<float>(), loss2.data_ptr<float>(), work.data_ptr(),
                                           wbytes, reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
    } else {
        check_status(fbw_b200_run(p.plan.data_ptr(), &p.summary, am_scores.data_ptr<float>(),
                                  out.data_ptr<float>(), sums.data_ptr<float>(), loss2.data_ptr<float>(),
                                  work.data_ptr(), wbytes,
                                  reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
    }
    return {out, sums, loss2};
}

// The op with the wrapper's passes folded in: log_probs (B,T,F) as the caller holds them ->
// [grad (B,T,F) = -posterior, sum_output (T,B)].  Replaces neg/transpose/contiguous before the op
// and neg/exp after it (i6_native_ops/fbw/__init__.py:41-44, 66); opt-in, used by fbw_loss_fused.
std::vector<torch::Tensor> fbw_fused(torch::Tensor& log_probs, torch::Tensor& edges,
                                     torch::Tensor& weights, torch::Tensor& start_end_states,
                                     torch::Tensor& seq_lens, int64_t num_states) {
    check_input(log_probs, torch::kFloat32, "log_probs");
    TORCH_CHECK(log_probs.dim() == 3, "log_probs must have shape (B, T, F)");
    TORCH_CHECK(start_end_states.dim() == 2 && start_end_states.size(1) == log_probs.size(0),
                "start_end_states must have shape (2, B) with B = log_probs.size(0)");
    check_input(edges, torch::kInt32, "edges");
    check_same_device(log_probs, edges);
    c10::cuda::CUDAGuard guard(log_probs.device());
    const int64_t B = log_probs.size(0), T = log_probs.size(1), F = log_probs.size(2);
    torch::Tensor grad = torch::empty_like(log_probs);
    torch::Tensor sums = torch::empty({T, B}, log_probs.options());
    Prepared p = prepare_impl(edges, weights, start_end_states, seq_lens, T, F, num_states);
    auto stream = at::cuda::getCurrentCUDAStream();
    size_t wbytes = fbw_b200_run_bytes(&p.summary);
    torch::Tensor work = byte_buffer(wbytes, log_probs.device());
    check_status(fbw_b200_run_fused(p.plan.data_ptr(), &p.summary, log_probs.data_ptr<float>(),
                                    grad.data_ptr<float>(), sums.data_ptr<float>(), nullptr,
                                    work.data_ptr(), wbytes,
                                    reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
    return {grad, sums};
}

// Two-step form of the same op for callers that reuse one batch of automata with new scores:
// fbw_prepare(...) -> opaque handle, fbw_run(handle, am_scores) -> [out, sum_output, loss2].
// loss2 = [sum of sum_output, sum over sequences of sum_output[0]].
struct PlanHandle {
    Prepared p;
    py::dict info() const {
        py::dict d;
        const fbw_b200_summary& s = p.summary;
        d["T"] = s.T; d["B"] = s.B; d["F"] = s.F; d["E"] = s.E; d["S"] = s.S;
        d["state_floats"] = s.state_floats; d["tiled_floats"] = s.tiled_floats;
        d["frame_floats"] = s.frame_floats; d["num_slots"] = s.num_slots;
        d["max_states"] = s.max_states; d["max_edges"] = s.max_edges;
        d["max_slots"] = s.max_slots; d["max_len"] = s.max_len; d["sum_len"] = s.sum_len;
        d["gather_units"] = s.gather_units; d["post_units"] = s.post_units;
        d["plan_bytes"] = (int64_t)p.plan.numel();
        d["run_bytes"] = (int64_t)fbw_b200_run_bytes(&s);
        return d;
    }
};

PlanHandle fbw_prepare(torch::Tensor& edges, torch::Tensor& weights,
                       torch::Tensor& start_end_states, torch::Tensor& seq_lens, int64_t T,
                       int64_t F, int64_t num_states) {
    TORCH_CHECK(edges.is_cuda(), "edges must be a CUDA tensor");
    c10::cuda::CUDAGuard guard(edges.device());
    PlanHandle h;
    h.p = prepare_impl(edges, weights, start_end_states, seq_lens, T, F, num_states);
    return h;
}

std::vector<torch::Tensor> fbw_run(const PlanHandle& h, torch::Tensor& am_scores) {
    check_input(am_scores, torch::kFloat32, "am_scores");
    const fbw_b200_summary& s = h.p.summary;
    TORCH_CHECK(am_scores.dim() == 3 && am_scores.size(0) == s.T && am_scores.size(1) == s.B &&
                    am_scores.size(2) == s.F,
                "am_scores must have the (T, B, F) the plan was prepared for");
    TORCH_CHECK(am_scores.device() == h.p.plan.device(), "am_scores and plan on different devices");
    c10::cuda::CUDAGuard guard(am_scores.device());
    return run_impl(h.p, am_scores, true);
}

// fbw_run with per-kernel device times: returns ([out, sum_output, loss2], [ms per phase]).
py::tuple fbw_run_phases(const PlanHandle& h, torch::Tensor& am_scores) {
    check_input(am_scores, torch::kFloat32, "am_scores");
    const fbw_b200_summary& s = h.p.summary;
    TORCH_CHECK(am_scores.dim() == 3 && am_scores.size(0) == s.T && am_scores.size(1) == s.B &&
                    am_scores.size(2) == s.F,
                "am_scores must have the (T, B, F) the plan was prepared for");
    c10::cuda::CUDAGuard guard(am_scores.device());
    auto stream = at::cuda::getCurrentCUDAStream();
    torch::Tensor out   = torch::empty_like(am_scores);
    torch::Tensor sums  = torch::empty({s.T, s.B}, am_scores.options());
    torch::Tensor loss2 = torch::empty({2}, am_scores.options());
    size_t wbytes = fbw_b200_run_bytes(&s);
    torch::Tensor work = byte_buffer(wbytes, am_scores.device());
    float ms[FBW_B200_NUM_PHASES];
    check_status(fbw_b200_run_phases(h.p.plan.data_ptr(), &s, am_scores.data_ptr<float>(),
                                     out.data_ptr<float>(), sums.data_ptr<float>(),
                                     loss2.data_ptr<float>(), work.data_ptr(), wbytes,
                                     reinterpret_cast<fbw_b200_stream_t>(stream.stream()), ms));
    py::list times;
    for (int i = 0; i < FBW_B200_NUM_PHASES; i++) times.append(ms[i]);
    py::list outs;
    outs.append(out); outs.append(sums); outs.append(loss2);
    return py::make_tuple(outs, times);
}

// Device-side automaton builders (no counterpart in the reference).  Both return the `fsa` tuple of
// fbw_loss / align_viterbi: (num_states, edges (4,E) int32, weights (E,) float32, start_end (2,B) int32).
py::tuple ctc_topology(torch::Tensor& labels, torch::Tensor& label_lens, int64_t blank) {
    check_input(labels, torch::kInt32, "labels");
    check_input(label_lens, torch::kInt32, "label_lens");
    TORCH_CHECK(labels.dim() == 2 && labels.size(0) > 0 && labels.size(1) > 0, "labels must have shape (B, Lmax)");
    TORCH_CHECK(label_lens.dim() == 1 && label_lens.size(0) == labels.size(0), "label_lens must have shape (B,)");
    c10::cuda::CUDAGuard guard(labels.device());
    auto stream = reinterpret_cast<fbw_b200_stream_t>(at::cuda::getCurrentCUDAStream().stream());
    const int64_t B = labels.size(0), Lmax = labels.size(1);
    size_t sbytes = fbw_b200_topology_bytes(B);
    torch::Tensor scratch = byte_buffer(sbytes, labels.device());
    int64_t S = 0, E = 0;
    check_status(fbw_b200_ctc_topology_count(labels.data_ptr<int32_t>(), label_lens.data_ptr<int32_t>(), B,
                                             Lmax, (int32_t)blank, scratch.data_ptr(), sbytes, &S, &E, stream));
    torch::Tensor edges     = torch::empty({4, E}, labels.options());
    torch::Tensor weights   = torch::empty({E}, labels.options().dtype(torch::kFloat32));
    torch::Tensor start_end = torch::empty({2, B}, labels.options());
    check_status(fbw_b200_ctc_topology_fill(labels.data_ptr<int32_t>(), label_lens.data_ptr<int32_t>(), B,
                                            Lmax, (int32_t)blank, scratch.data_ptr(), E,
                                            edges.data_ptr<int32_t>(), weights.data_ptr<float>(),
                                            start_end.data_ptr<int32_t>(), stream));
    return py::make_tuple(S, edges, weights, start_end);
}

py::tuple hmm_topology(torch::Tensor& classes, torch::Tensor& lens, c10::optional<torch::Tensor> optional,
                       double loop_weight, double forward_weight, c10::optional<double> skip_weight) {
    check_input(classes, torch::kInt32, "classes");
    check_input(lens, torch::kInt32, "lens");
    TORCH_CHECK(classes.dim() == 2 && classes.size(0) > 0 && classes.size(1) > 0, "classes must have shape (B, Nmax)");
    TORCH_CHECK(lens.dim() == 1 && lens.size(0) == classes.size(0), "lens must have shape (B,)");
    const uint8_t* opt = nullptr;
    if (optional.has_value()) {
        check_input(*optional, torch::kUInt8, "optional");
        TORCH_CHECK(optional->sizes() == classes.sizes(), "optional must have the shape of classes");
        opt = optional->data_ptr<uint8_t>();
    }
    c10::cuda::CUDAGuard guard(classes.device());
    auto stream = reinterpret_cast<fbw_b200_stream_t>(at::cuda::getCurrentCUDAStream().stream());
    const int64_t B = classes.size(0), Nmax = classes.size(1);
    const int skip_all = skip_weight.has_value() ? 1 : 0;
    size_t sbytes = fbw_b200_topology_bytes(B);
    torch::Tensor scratch = byte_buffer(sbytes, classes.device());
    int64_t S = 0, E = 0;
    check_status(fbw_b200_hmm_topology_count(lens.data_ptr<int32_t>(), opt, B, Nmax, skip_all,
                                             scratch.data_ptr(), sbytes, &S, &E, stream));
    TORCH_CHECK(E > 0, "hmm_topology: no sequence has a state");
    torch::Tensor edges     = torch::empty({4, E}, classes.options());
    torch::Tensor weights   = torch::empty({E}, classes.options().dtype(torch::kFloat32));
    torch::Tensor start_end = torch::empty({2, B}, classes.options());
    check_status(fbw_b200_hmm_topology_fill(classes.data_ptr<int32_t>(), lens.data_ptr<int32_t>(), opt, B, Nmax,
                                            (float)loop_weight, (float)forward_weight,
                                            (float)skip_weight.value_or(0.0), skip_all, scratch.data_ptr(),
                                            E, edges.data_ptr<int32_t>(), weights.data_ptr<float>(),
                                            start_end.data_ptr<int32_t>(), stream));
    return py::make_tuple(S, edges, weights, start_end);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("ctc_topology", &ctc_topology, "CTC automata of a batch of label sequences, built on the device");
    m.def("hmm_topology", &hmm_topology, "Left-to-right HMM automata of a batch of class sequences",
          py::arg("classes"), py::arg("lens"), py::arg("optional") = py::none(), py::arg("loop_weight"),
          py::arg("forward_weight"), py::arg("skip_weight") = py::none());
    m.def("fbw_run_phases", &fbw_run_phases, "fbw_run with per-kernel device times");
    m.def("launch_count", []() { return fbw_b200_launch_count(); });
    m.def("fbw", &fbw, "Fast Baum-Welch CUDA routine (B200)");
    m.def("fbw_fused", &fbw_fused, "fbw on (B,T,F) log_probs, returning the gradient directly");
    m.def("fbw_host_scores", &fbw_host_scores,
          "fbw on scores in pinned host memory: only the scores the automata need cross the bus; "
          "`out`: optional pinned host tensor that receives the (T,B,F) result directly",
          py::arg("am_scores"), py::arg("edges"), py::arg("weights"), py::arg("start_end_states"),
          py::arg("seq_lens"), py::arg("num_states"), py::arg("out") = py::none(), py::arg("staged") = true);
    m.def("fbw_prepare", &fbw_prepare, "Validate and sort a batch of automata");
    m.def("fbw_run", &fbw_run, "Run fbw on prepared automata");
    m.def("abi_version", []() { return fbw_b200_abi_version(); });

    py::class_<DebugOptions>(m, "DebugOptions", py::module_local())
        .def(py::init<>())
        .def_readwrite("dump_alignment", &DebugOptions::dump_alignment)
        .def_readwrite("dump_output", &DebugOptions::dump_output)
        .def_readwrite("dump_every", &DebugOptions::dump_every)
        .def_readwrite("pruning", &DebugOptions::pruning);

    py::class_<PlanHandle>(m, "PlanHandle", py::module_local()).def("info", &PlanHandle::info);
}
