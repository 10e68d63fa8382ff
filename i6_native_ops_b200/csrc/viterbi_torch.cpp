// viterbi_torch.cpp -- torch extension `fast_viterbi_core`: the Python-visible best-path op over
// the C ABI of include/fbw_b200.h.  Mirrors the reference binding
// i6_native_ops/fast_viterbi/binding.cpp:13-29: one member `fast_viterbi` with the same six
// positional arguments, the same input checks (CUDA, contiguous, dtype -> RuntimeError) and the same
// two outputs [alignment (T,B) int32, scores (B,) float32].
//
// Differences that do not change results: scratch comes from torch's caching allocator instead of
// device_malloc / device_free per call (core.cu:216, 244, 269-270); work is enqueued on torch's
// current stream of the inputs' device under a device guard; malformed automata raise RuntimeError
// instead of being undefined behaviour.
#include <torch/extension.h>

#include <vector>

#include "fbw_b200.h"
#include "torch_common.h"

using namespace fbw_b200::torch_glue;

namespace {

std::vector<torch::Tensor> viterbi_impl(const torch::Tensor& scores_in, const torch::Tensor& edges,
                                        const torch::Tensor& weights,
                                        const torch::Tensor& start_end_states,
                                        const torch::Tensor& seq_lens, int64_t num_states,
                                        bool batch_major, bool host_scores = false) {
    if (host_scores) {
        TORCH_CHECK(!scores_in.is_cuda() && scores_in.is_pinned(),
                    "scores must be a pinned host tensor (use fast_viterbi() for CUDA tensors)");
        TORCH_CHECK(scores_in.is_contiguous() && scores_in.scalar_type() == torch::kFloat32,
                    "scores must be contiguous float32");
        TORCH_CHECK(edges.is_cuda(), "edges must be a CUDA tensor");
    } else {
        check_input(scores_in, torch::kFloat32, batch_major ? "log_probs" : "am_scores");
        check_input(edges, torch::kInt32, "edges");
        check_same_device(scores_in, edges);
    }
    TORCH_CHECK(scores_in.dim() == 3, "scores must have three dimensions");
    const int64_t B = scores_in.size(batch_major ? 0 : 1), T = scores_in.size(batch_major ? 1 : 0);
    const int64_t F = scores_in.size(2);
    TORCH_CHECK(start_end_states.dim() == 2 && start_end_states.size(1) == B,
                "start_end_states must have shape (2, B) with B the batch size of the scores");
    c10::cuda::CUDAGuard guard(edges.device());
    auto int_opts = edges.options();      // int32 on the automata's device
    auto f32_opts = weights.options();    // float32 on the automata's device
    torch::Tensor alignment = batch_major ? torch::empty({B, T}, int_opts) : torch::empty({T, B}, int_opts);
    torch::Tensor scores    = torch::empty({B}, f32_opts);
    Prepared p = prepare_impl(edges, weights, start_end_states, seq_lens, T, F, num_states);
    auto   stream = at::cuda::getCurrentCUDAStream();
    size_t wbytes = fbw_b200_viterbi_bytes(&p.summary);
    torch::Tensor work = byte_buffer(wbytes, edges.device());
    // large calls on scores in host memory with few classes per sequence: host threads of the library
    // pick the scores the automata need out of the pinned tensor instead of 32-byte reads over the bus
    if (host_scores && (double)scores_in.numel() >= 1.0e7 && p.summary.max_slots * 16 <= p.summary.F) {
        const size_t hbytes = fbw_b200_run_with_host_bytes(&p.summary);
        torch::Tensor host_work = torch::empty({(int64_t)hbytes}, torch::TensorOptions().dtype(torch::kUInt8).pinned_memory(true));
        check_status(fbw_b200_viterbi_with_host(p.plan.data_ptr(), &p.summary, scores_in.data_ptr<float>(),
                                                alignment.data_ptr<int32_t>(), scores.data_ptr<float>(),
                                                batch_major ? 1 : 0, work.data_ptr(), wbytes, host_work.data_ptr(),
                                                hbytes, reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
        return {alignment, scores};
    }
    check_status(fbw_b200_viterbi(p.plan.data_ptr(), &p.summary, scores_in.data_ptr<float>(),
                                  alignment.data_ptr<int32_t>(), scores.data_ptr<float>(),
                                  batch_major ? 1 : 0, work.data_ptr(), wbytes,
                                  reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
    return {alignment, scores};
}

}  // namespace

// The op.  Signature and meaning of the reference's fast_viterbi() (binding.cpp:13-25): am_scores
// (T,B,F) f32 positive log scores, edges (4,E) i32, weights (E) f32, start_end_states (2,B) i32,
// seq_lens (B) i32, num_states -> [alignment (T,B) i32, scores (B) f32].
std::vector<torch::Tensor> fast_viterbi(torch::Tensor& am_scores, torch::Tensor& edges,
                                        torch::Tensor& weights, torch::Tensor& start_end_states,
                                        torch::Tensor& seq_lens, unsigned num_states) {
    return viterbi_impl(am_scores, edges, weights, start_end_states, seq_lens, (int64_t)num_states,
                        false);
}

// The op with the wrapper's transposes folded in (i6_native_ops/fast_viterbi/__init__.py:37, 46):
// log_probs (B,T,F) as the caller holds them -> [alignment (B,T) i32, scores (B) f32].
std::vector<torch::Tensor> fast_viterbi_batch_major(torch::Tensor& log_probs, torch::Tensor& edges,
                                                    torch::Tensor& weights,
                                                    torch::Tensor& start_end_states,
                                                    torch::Tensor& seq_lens, int64_t num_states) {
    return viterbi_impl(log_probs, edges, weights, start_end_states, seq_lens, num_states, true);
}

// fast_viterbi on scores in PINNED HOST memory (a pinned CPU tensor, (T,B,F)): the gather kernel reads
// the scores the automata need straight out of host memory through the unified address space instead
// of the whole tensor being copied to the device first.  Same results.  No counterpart in the
// reference, which requires CUDA tensors (binding.cpp:16-20).
std::vector<torch::Tensor> fast_viterbi_host_scores(torch::Tensor& am_scores, torch::Tensor& edges,
                                                    torch::Tensor& weights,
                                                    torch::Tensor& start_end_states,
                                                    torch::Tensor& seq_lens, int64_t num_states) {
    return viterbi_impl(am_scores, edges, weights, start_end_states, seq_lens, num_states, false, true);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("fast_viterbi_host_scores", &fast_viterbi_host_scores,
          "fast_viterbi on scores in pinned host memory: only the scores the automata need cross the bus");
    m.def("fast_viterbi", &fast_viterbi, "Fast Viterbi CUDA routine (B200)");
    m.def("fast_viterbi_batch_major", &fast_viterbi_batch_major,
          "fast_viterbi on (B,T,F) log_probs, returning the (B,T) alignment directly");
    m.def("launch_count", []() { return fbw_b200_launch_count(); });
}
