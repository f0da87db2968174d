// Constants and launcher prototypes shared by the kernel and the host translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fkb {

struct LaunchParams;

constexpr uint32_t kStagedThreads = 256;
// Shared memory of one staged CTA: a 1 KB header (mbarriers, tile infos, plane records), two source buffers
// and two output buffers.  111 KB in total, so two CTAs fit in the 228 KB of an SM.
constexpr uint32_t kInBytes = 32 * 1024;
constexpr uint32_t kOutBytes = 23 * 1024;
constexpr uint32_t kStagedSmemBytes = 1024 + 2 * (kInBytes + kOutBytes);

cudaError_t launch_staged(const LaunchParams& p, uint32_t grid, cudaStream_t stream);
cudaError_t launch_gather(const LaunchParams& p, dim3 grid, cudaStream_t stream);
cudaError_t status_word_address(int** out);

}  // namespace fkb
