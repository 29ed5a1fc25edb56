// Head-slice interleave for the multi-GPU gather: the collective lands the
// ranks' attention outputs rank-major, [world][rows][slice] (slice = the rank's
// heads * 128 columns); the caller of the attention path expects token-major
// [rows][world*slice].  One 16-byte vector per thread, grid-stride.

#include <cuda_runtime.h>
#include <stdint.h>

#include "../qw_cuda.h"

namespace {

__global__ void __launch_bounds__(256)
qw_interleave_kernel(uint4 *__restrict__ full, const uint4 *__restrict__ staged, uint32_t rows,
                     uint32_t slice_vecs, uint32_t world) {
    const size_t total = (size_t)rows * slice_vecs * world;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        // i enumerates the destination: (row, rank, vec)
        const uint32_t vec = (uint32_t)(i % slice_vecs);
        const size_t t = i / slice_vecs;
        const uint32_t rank = (uint32_t)(t % world);
        const size_t row = t / world;
        full[i] = staged[((size_t)rank * rows + row) * slice_vecs + vec];
    }
}

}  // namespace

extern "C" int qwcu_interleave_launch(void *full, const void *staged, uint32_t rows,
                                      uint32_t slice_elements, uint32_t world, int sm_count,
                                      qwcu_stream stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (slice_elements % 8) return (int)cudaErrorInvalidValue;
    const uint32_t slice_vecs = slice_elements / 8;
    const size_t total = (size_t)rows * slice_vecs * world;
    if (!total) return 0;
    size_t want = (total + 255) / 256;
    size_t cap = (size_t)(sm_count > 0 ? sm_count : 148) * 8;
    unsigned int blocks = (unsigned int)(want < cap ? want : cap);
    qw_interleave_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint4 *>(full),
                                                     static_cast<const uint4 *>(staged), rows,
                                                     slice_vecs, world);
    return (int)cudaGetLastError();
}
