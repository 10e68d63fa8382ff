// torch_common.h -- what the torch extensions over the C ABI of include/fbw_b200.h share: input
// checks in the style of the reference's CHECK_INPUT (i6_native_ops/common/returnn_definitions.h:93-99,
// device / layout / dtype -> RuntimeError), status-code conversion, scratch from torch's caching
// allocator, and the validated plan of a batch of automata.
#pragma once

#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "fbw_b200.h"

namespace fbw_b200 {
namespace torch_glue {

inline void check_input(const torch::Tensor& x, torch::ScalarType dtype, const char* name) {
    TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(x.scalar_type() == dtype, name, " must have dtype ", dtype);
}

// device scores must live where the automata live
inline void check_same_device(const torch::Tensor& scores, const torch::Tensor& edges) {
    TORCH_CHECK(scores.device() == edges.device(),
                "the scores and the automaton tensors must be on the same device");
}

inline void check_status(int status, const fbw_b200_summary* s = nullptr) {
    if (status == FBW_B200_OK) return;
    if (status == FBW_B200_BAD_AUTOMATON && s) {
        TORCH_CHECK(false, "fbw: ", fbw_b200_status_string(status), " (validation bits ", s->error,
                    ")");
    }
    if (status == FBW_B200_CUDA_ERROR) {
        TORCH_CHECK(false, "fbw: CUDA error: ", cudaGetErrorString(cudaGetLastError()));
    }
    TORCH_CHECK(false, "fbw: ", fbw_b200_status_string(status));
}

inline torch::Tensor byte_buffer(size_t bytes, const torch::Device& dev) {
    return torch::empty({(int64_t)(bytes > 0 ? bytes : 1)},
                        torch::TensorOptions().dtype(torch::kUInt8).device(dev));
}

struct Prepared {
    torch::Tensor    plan;
    fbw_b200_summary summary;
};

inline Prepared prepare_impl(const torch::Tensor& edges, const torch::Tensor& weights,
                      const torch::Tensor& start_end_states, const torch::Tensor& seq_lens,
                      int64_t T, int64_t F, int64_t num_states) {
    check_input(edges, torch::kInt32, "edges");
    check_input(weights, torch::kFloat32, "weights");
    check_input(start_end_states, torch::kInt32, "start_end_states");
    check_input(seq_lens, torch::kInt32, "seq_lens");
    TORCH_CHECK(edges.dim() == 2 && edges.size(0) == 4, "edges must have shape (4, E)");
    const int64_t E = edges.size(1);
    TORCH_CHECK(weights.dim() == 1 && weights.size(0) == E, "weights must have shape (E,)");
    TORCH_CHECK(start_end_states.dim() == 2 && start_end_states.size(0) == 2,
                "start_end_states must have shape (2, B)");
    const int64_t B = start_end_states.size(1);
    TORCH_CHECK(seq_lens.dim() == 1 && seq_lens.size(0) == B, "seq_lens must have shape (B,)");
    TORCH_CHECK(T > 0 && B > 0 && F > 0, "am_scores must be non-empty");
    // a kernel given another GPU's pointer faults (or, with peer access, silently reads remote memory)
    TORCH_CHECK(weights.device() == edges.device() && start_end_states.device() == edges.device() &&
                    seq_lens.device() == edges.device(),
                "edges, weights, start_end_states and seq_lens must be on the same device");
    TORCH_CHECK(num_states > 0, "num_states must be positive");

    auto   stream = at::cuda::getCurrentCUDAStream();
    size_t pbytes = fbw_b200_plan_bytes(B, E, num_states);
    Prepared p;
    p.plan = byte_buffer(pbytes, edges.device());
    check_status(fbw_b200_prepare(edges.data_ptr<int32_t>(), weights.data_ptr<float>(),
                                  start_end_states.data_ptr<int32_t>(),
                                  seq_lens.data_ptr<int32_t>(), T, B, F, E, num_states,
                                  p.plan.data_ptr(), pbytes,
                                  reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
    int st = fbw_b200_plan_summary(p.plan.data_ptr(), &p.summary,
                                   reinterpret_cast<fbw_b200_stream_t>(stream.stream()));
    if (st == FBW_B200_RETRY_GENERAL) {  // a sequence too large for the fast plan builder
        check_status(fbw_b200_prepare_general(
            edges.data_ptr<int32_t>(), weights.data_ptr<float>(),
            start_end_states.data_ptr<int32_t>(), seq_lens.data_ptr<int32_t>(), T, B, F, E,
            num_states, p.plan.data_ptr(), pbytes,
            reinterpret_cast<fbw_b200_stream_t>(stream.stream())));
        st = fbw_b200_plan_summary(p.plan.data_ptr(), &p.summary,
                                   reinterpret_cast<fbw_b200_stream_t>(stream.stream()));
    }
    check_status(st, &p.summary);
    return p;
}

}  // namespace torch_glue
}  // namespace fbw_b200
