// Internal: host-side launchers implemented by the kernel translation units.
#pragma once
#include <cuda_runtime.h>

namespace dfa3d {
struct KArgs;
// mode: dfa3d::Mode
cudaError_t launch_forward(const KArgs &a, bool value_bf16, bool dist_bf16, int mode, cudaStream_t s);
cudaError_t launch_depth_score_forward(const KArgs &a, bool dist_bf16, cudaStream_t s);
cudaError_t launch_backward(const KArgs &a, bool value_bf16, bool dist_bf16, int mode, cudaStream_t s);
cudaError_t launch_depth_score_backward(const KArgs &a, bool dist_bf16, cudaStream_t s);
}  // namespace dfa3d
