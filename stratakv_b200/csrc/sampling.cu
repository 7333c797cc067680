// Next-token choice on the device: greedy argmax and a finite check of the logits.
//
// The reference copies the whole logits row to the host and samples there
// (src/generation/generator.cpp:716-739, src/generation/sampler.cpp:43-148); here
// only the chosen ids cross.  Greedy: the largest logit, the lowest index among
// equals (src/generation/sampler.cpp:58-62).
#include "common.cuh"

namespace skv {

// One block per row.  flag |= 2 if a logit of the row is NaN or infinite
// (src/generation/sampler.cpp:52-56 rejects such rows).
__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab,
                              int* __restrict__ flag) {
    __shared__ float best_value[32];
    __shared__ int best_index[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float value = -INFINITY;
    int index = 0x7fffffff;
    bool bad = false;
    for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
        const float v = row[c];
        if (!isfinite(v)) bad = true;
        if (v > value || (v == value && c < index)) { value = v; index = c; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other_value > value || (other_value == value && other_index < index)) {
            value = other_value; index = other_index;
        }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0 && flag) atomicOr(flag, 2);
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (warp == 0) {
        value = lane < warps ? best_value[lane] : -INFINITY;
        index = lane < warps ? best_index[lane] : 0x7fffffff;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
            const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
            if (other_value > value || (other_value == value && other_index < index)) {
                value = other_value; index = other_index;
            }
        }
        if (lane == 0) out[blockIdx.x] = index == 0x7fffffff ? 0 : index;
    }
}

}  // namespace skv

using namespace skv;

SKV_EXPORT int skv_argmax(const float* logits, int* out, int rows, int vocab, int* flag, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fail("skv_argmax", "vocab must be positive");
    argmax_kernel<<<rows, 256, 0, stream>>>(logits, out, vocab, flag);
    return check_launch("skv_argmax");
}
