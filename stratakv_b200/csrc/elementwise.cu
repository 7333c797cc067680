// Embedding gather, RMSNorm, rotary encoding with cache write, residual helpers.
//
// These replace the reference's embedding_lookup_kernel, rmsnorm_kernel,
// generate_rope_frequencies_kernel + rope_split_half_kernel and the two
// device-to-device copies that append K and V (src/cuda/gemm_cuda.cu:172-202,
// 239-274, 286-295; src/models/transformer_block.cpp:484-509), for a batch of
// tokens instead of one, and without --use_fast_math: 1/sqrtf and a host-built
// cos/sin table stand where the reference has rsqrtf and fast sincosf.
#include "common.cuh"

namespace skv {

// ---------------------------------------------------------------------------
// x[t, :] = table[ids[t], :] widened to float.  An id outside the vocabulary
// (hosts check before launching) writes zeros and raises the flag.
// With `scaled` the row times `gamma_next` is left at scaled[t, :], its sum of squares at partials[t * stride]
// (one partial sum) and the factor 1 / sqrt(mean(row^2) + eps_next) at row_scale[t], for the projection
// after the first norm (see linear.cu).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, int vocab, int* __restrict__ flag,
                             float* __restrict__ row_scale, const float* __restrict__ gamma_next, float eps_next,
                             T* __restrict__ scaled, float* __restrict__ partials, int stride) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* row_out = out + (size_t)t * hidden;
    const bool bad = id < 0 || id >= vocab;
    if (bad && threadIdx.x == 0 && flag) atomicOr(flag, 1);
    const T* row = table + (size_t)(bad ? 0 : id) * hidden;
    float partial = 0.0f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = bad ? 0.0f : to_float(row[c]);
        row_out[c] = v;
        if (scaled) {
            partial = fmaf(v, v, partial);
            scaled[(size_t)t * hidden + c] = from_float<T>(v * gamma_next[c]);
        }
    }
    if (scaled) {
        const float total = block_sum(partial, scratch);
        if (threadIdx.x == 0) {
            partials[(size_t)t * stride] = total;
            row_scale[t] = 1.0f / sqrtf(total / (float)hidden + eps_next);
        }
    }
}

// ---------------------------------------------------------------------------
// y[r, :] = x[src(r), :] * (1 / sqrt(mean(x^2) + eps)) * gamma, sums in float.
// The multiplication order is the reference's (src/layers/rmsnorm.cpp:91-93).
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                               float eps, T* __restrict__ out, const int* __restrict__ rows,
                               int hidden) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float* row = x + (size_t)src * hidden;
    float partial = 0.0f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = row[c];
        partial = fmaf(v, v, partial);
    }
    const float mean_square = block_sum(partial, scratch) / (float)hidden;
    const float inverse_rms = 1.0f / sqrtf(mean_square + eps);
    T* row_out = out + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        row_out[c] = from_float<T>(row[c] * inverse_rms * gamma[c]);
}

// The same with one warp per row and 16-byte loads, for steps with many rows (hidden % 4 == 0):
// the row is read twice, the second time from L1.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ gamma, float eps,
                    T* __restrict__ out, const int* __restrict__ rows, int n_rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const int src = rows ? rows[r] : r;
    const float4* row = (const float4*)(x + (size_t)src * hidden);
    const int quads = hidden >> 2;
    // The first 2,048 columns of the row stay in registers: all their loads are in flight at once and nothing of
    // them is read again.  A longer row's remainder is read twice, as the whole row was before.
    constexpr int HELD = 16;
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 held[HELD];
#pragma unroll
    for (int j = 0; j < HELD; ++j) held[j] = lane + 32 * j < quads ? row[lane + 32 * j] : zero;
    float partial[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < HELD; ++j) {
        partial[0] = fmaf(held[j].x, held[j].x, partial[0]); partial[1] = fmaf(held[j].y, held[j].y, partial[1]);
        partial[2] = fmaf(held[j].z, held[j].z, partial[2]); partial[3] = fmaf(held[j].w, held[j].w, partial[3]);
    }
    for (int i = lane + 32 * HELD; i < quads; i += 32) {
        const float4 v = row[i];
        partial[0] = fmaf(v.x, v.x, partial[0]); partial[1] = fmaf(v.y, v.y, partial[1]);
        partial[2] = fmaf(v.z, v.z, partial[2]); partial[3] = fmaf(v.w, v.w, partial[3]);
    }
    const float mean_square = warp_sum((partial[0] + partial[1]) + (partial[2] + partial[3])) / (float)hidden;
    const float inverse_rms = 1.0f / sqrtf(mean_square + eps);
    T* row_out = out + (size_t)r * hidden;
    const float4* g4 = (const float4*)gamma;
    auto emit = [&](int i, const float4& v) {
        const float4 g = g4[i];
        const float y0 = v.x * inverse_rms * g.x, y1 = v.y * inverse_rms * g.y;
        const float y2 = v.z * inverse_rms * g.z, y3 = v.w * inverse_rms * g.w;
        if (sizeof(T) == 4) {
            ((float4*)row_out)[i] = make_float4(y0, y1, y2, y3);
        } else {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
            ((uint2*)row_out)[i] = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
        }
    };
#pragma unroll
    for (int j = 0; j < HELD; ++j)
        if (lane + 32 * j < quads) emit(lane + 32 * j, held[j]);
    for (int i = lane + 32 * HELD; i < quads; i += 32) emit(i, row[i]);
}

// ---------------------------------------------------------------------------
// One token per block.  Rotates every query head and key head with split-half
// pairs (i, i + head_dim/2) (src/layers/attention.cpp:96-135), writes queries
// in the compute dtype, and writes the rotated keys and the values into the
// token's place in the paged cache: block = table[seq][pos / block_size],
// row = pos % block_size of tile [kv_head][block_size][head_dim].
template <typename T>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, const float2* __restrict__ cos_sin,
                                     const int* __restrict__ positions, const int* __restrict__ token_seq,
                                     const int* __restrict__ block_table, int table_width,
                                     T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     int num_heads, int num_kv_heads, int head_dim, int block_size,
                                     int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const int q_dim = num_heads * head_dim, kv_dim = num_kv_heads * head_dim;
    const int pos = positions[t];
    const float* src = qkv + (size_t)t * (q_dim + 2 * kv_dim);
    const float2* angles = cos_sin ? cos_sin + (size_t)pos * half : nullptr;
    size_t tile_base = 0;
    if (write_kv) {
        const int seq = token_seq[t];
        const int block = block_table[(size_t)seq * table_width + pos / block_size];
        tile_base = ((size_t)block * num_kv_heads * block_size + (pos % block_size)) * head_dim;
    }
    const int rotary_heads = num_heads + (write_kv ? num_kv_heads : 0);
    for (int idx = threadIdx.x; idx < rotary_heads * half; idx += blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        const float* x = src + (size_t)head * head_dim;     // key heads follow the query heads
        float c = 1.0f, s = 0.0f;
        if (angles) { const float2 a = angles[i]; c = a.x; s = a.y; }
        const float x1 = x[i], x2 = x[i + half];
        const float r1 = x1 * c - x2 * s;
        const float r2 = x1 * s + x2 * c;
        if (head < num_heads) {
            T* dst = q_out + (size_t)t * q_dim + (size_t)head * head_dim;
            dst[i] = from_float<T>(r1);
            dst[i + half] = from_float<T>(r2);
        } else {
            const int g = head - num_heads;
            T* dst = k_cache + tile_base + (size_t)g * block_size * head_dim;
            dst[i] = from_float<T>(r1);
            dst[i + half] = from_float<T>(r2);
        }
    }
    if (write_kv) {
        const float* v = src + q_dim + kv_dim;
        for (int idx = threadIdx.x; idx < kv_dim; idx += blockDim.x) {
            const int g = idx / head_dim, d = idx - g * head_dim;
            v_cache[tile_base + (size_t)g * block_size * head_dim + d] = from_float<T>(v[idx]);
        }
    }
}

// The same with four pairs (and four values) per thread and 16-byte loads; head_dim % 8 == 0.
template <typename T>
__device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d) {
    if (sizeof(T) == 4) {
        *(float4*)dst = make_float4(a, b, c, d);
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        *(uint2*)dst = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_vec_kernel(const float* __restrict__ qkv, const float2* __restrict__ cos_sin,
                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ block_table, int table_width, T* __restrict__ q_out,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, int num_heads, int num_kv_heads,
                         int head_dim, int block_size, int write_kv, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    // a warp per token, four tokens per block: a grid of one small block per token takes longer to start than to run
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n_tokens) return;
    const int half = head_dim >> 1, quads = half >> 2;
    const int q_dim = num_heads * head_dim, kv_dim = num_kv_heads * head_dim;
    const int pos = positions[t];
    const float* src = qkv + (size_t)t * (q_dim + 2 * kv_dim);
    const float4* angles = cos_sin ? (const float4*)(cos_sin + (size_t)pos * half) : nullptr;
    size_t tile_base = 0;
    if (write_kv) {
        const int seq = token_seq[t];
        const int block = block_table[(size_t)seq * table_width + pos / block_size];
        tile_base = ((size_t)block * num_kv_heads * block_size + (pos % block_size)) * head_dim;
    }
    const int rotary_heads = num_heads + (write_kv ? num_kv_heads : 0);
    // four items per lane and round: their loads go out together, then the four are rotated and stored
    const int items = rotary_heads * quads;
    for (int first = lane; first < items; first += 128) {
        float4 x1[4], x2[4], c[4], sn[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = first + 32 * u;
            if (idx < items) {
                const int head = idx / quads, i = (idx - head * quads) << 2;
                const float* x = src + (size_t)head * head_dim;
                x1[u] = *(const float4*)(x + i);
                x2[u] = *(const float4*)(x + i + half);
                c[u] = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                sn[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (angles) {
                    const float4 a = angles[i >> 1], b = angles[(i >> 1) + 1];      // (cos, sin) pairs i..i+1 and i+2..i+3
                    c[u] = make_float4(a.x, a.z, b.x, b.z);
                    sn[u] = make_float4(a.y, a.w, b.y, b.w);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = first + 32 * u;
            if (idx < items) {
                const int head = idx / quads, i = (idx - head * quads) << 2;
                T* dst = head < num_heads ? q_out + (size_t)t * q_dim + (size_t)head * head_dim
                                          : k_cache + tile_base + (size_t)(head - num_heads) * block_size * head_dim;
                store4<T>(dst + i, x1[u].x * c[u].x - x2[u].x * sn[u].x, x1[u].y * c[u].y - x2[u].y * sn[u].y,
                          x1[u].z * c[u].z - x2[u].z * sn[u].z, x1[u].w * c[u].w - x2[u].w * sn[u].w);
                store4<T>(dst + i + half, x1[u].x * sn[u].x + x2[u].x * c[u].x, x1[u].y * sn[u].y + x2[u].y * c[u].y,
                          x1[u].z * sn[u].z + x2[u].z * c[u].z, x1[u].w * sn[u].w + x2[u].w * c[u].w);
            }
        }
    }
    if (write_kv) {
        const float* v = src + q_dim + kv_dim;
        for (int idx = lane; idx < kv_dim >> 2; idx += 32) {
            const int e = idx << 2, g = e / head_dim, d = e - g * head_dim;
            const float4 value = *(const float4*)(v + e);
            store4<T>(v_cache + tile_base + (size_t)g * block_size * head_dim + d, value.x, value.y, value.z, value.w);
        }
    }
}

// out[i] += in[i]  (float residual stream; used by parts that have no fused epilogue)
__global__ void add_inplace_kernel(float* __restrict__ out, const float* __restrict__ in, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] += in[i];
}

}  // namespace skv

using namespace skv;

SKV_EXPORT const char* skv_last_error() { return error_buffer(); }
SKV_EXPORT int skv_library_dtype() { return SKV_DTYPE; }
SKV_EXPORT int skv_library_head_dim() { return SKV_HEAD_DIM; }

// Checkpoint tensors in the stored type -> the type a part computes in, on the device (the reference converts
// FP32 weights to BF16 by dropping the low half, src/cuda/gemm_cuda.cu:74-83; here to nearest even).  Kinds: 0 float32,
// 1 bfloat16, 2 float16.  The same in every build of the library.
template <int KIND> struct StoredType;
template <> struct StoredType<0> { typedef float type; };
template <> struct StoredType<1> { typedef __nv_bfloat16 type; };
template <> struct StoredType<2> { typedef __half type; };
__device__ __forceinline__ float stored_to_float(float v) { return v; }
__device__ __forceinline__ float stored_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float stored_to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ void float_to_stored(float v, float* out) { *out = v; }
__device__ __forceinline__ void float_to_stored(float v, __nv_bfloat16* out) { *out = __float2bfloat16_rn(v); }
__device__ __forceinline__ void float_to_stored(float v, __half* out) { *out = __float2half_rn(v); }

template <typename From, typename To>
__global__ void __launch_bounds__(256) convert_kernel(const From* __restrict__ src, To* __restrict__ dst, size_t count) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
        float_to_stored(stored_to_float(src[i]), dst + i);
}

template <int FROM>
static int launch_convert(const void* src, void* dst, int to, size_t count, cudaStream_t stream) {
    typedef typename StoredType<FROM>::type From;
    const size_t wanted = (count + 255) / 256;
    const dim3 grid((unsigned)(wanted < 65535 ? wanted : 65535));
    if (to == 0) convert_kernel<From, float><<<grid, 256, 0, stream>>>((const From*)src, (float*)dst, count);
    else if (to == 1) convert_kernel<From, __nv_bfloat16><<<grid, 256, 0, stream>>>((const From*)src, (__nv_bfloat16*)dst, count);
    else convert_kernel<From, __half><<<grid, 256, 0, stream>>>((const From*)src, (__half*)dst, count);
    const cudaError_t status = cudaGetLastError();
    return status == cudaSuccess ? 0 : fail("skv_convert", cudaGetErrorString(status));
}

SKV_EXPORT int skv_convert(const void* src, int from, void* dst, int to, long long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (from < 0 || from > 2 || to < 0 || to > 2) return fail("skv_convert", "types are 0 float32, 1 bfloat16, 2 float16");
    if (from == 0) return launch_convert<0>(src, dst, to, (size_t)count, stream);
    if (from == 1) return launch_convert<1>(src, dst, to, (size_t)count, stream);
    return launch_convert<2>(src, dst, to, (size_t)count, stream);
}

SKV_EXPORT int skv_embed(const void* table, const int* ids, float* out, int n_tokens, int hidden,
                         int vocab, int* flag, void* scaled, const float* gamma_next, float* partials,
                         int partial_stride, float* row_scale, float eps_next, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return fail("skv_embed", "hidden and vocab must be positive");
    if (scaled && (!gamma_next || !partials || !row_scale || partial_stride < 1))
        return fail("skv_embed", "the next norm's weight and places for the sums of squares and the factors are needed");
    const int threads = hidden >= 1024 ? 256 : 128;
    return launch_pdl("skv_embed", embed_kernel<skv_t>, dim3(n_tokens), dim3(threads), 0, stream,
                      (const skv_t*)table, ids, out, hidden, vocab, flag, row_scale, gamma_next, eps_next,
                      (skv_t*)scaled, partials, partial_stride);
}

SKV_EXPORT int skv_rmsnorm(const float* x, const float* gamma, float eps, void* out, const int* rows,
                           int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (hidden <= 0) return fail("skv_rmsnorm", "hidden must be positive");
    // a warp per row once there are rows enough to fill the GPU that way, else a block per row
    if (n_rows >= 1024 && hidden % 4 == 0 && (((uintptr_t)x | (uintptr_t)gamma | (uintptr_t)out) & 15) == 0)
        return launch_pdl("skv_rmsnorm", rmsnorm_rows_kernel<skv_t>, dim3((n_rows + 7) / 8), dim3(256), 0, stream, x,
                          gamma, eps, (skv_t*)out, rows, n_rows, hidden);
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return launch_pdl("skv_rmsnorm", rmsnorm_kernel<skv_t>, dim3(n_rows), dim3(threads), 0, stream, x, gamma, eps,
                      (skv_t*)out, rows, hidden);
}

SKV_EXPORT int skv_rope_kv_write(const float* qkv, const float* cos_sin, const int* positions,
                                 const int* token_seq, const int* block_table, int table_width,
                                 void* q_out, void* k_cache, void* v_cache, int n_tokens,
                                 int num_heads, int num_kv_heads, int head_dim, int block_size,
                                 int write_kv, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || (head_dim & 1)) return fail("skv_rope_kv_write", "head_dim must be positive and even");
    if (num_heads <= 0 || num_kv_heads <= 0 || block_size <= 0)
        return fail("skv_rope_kv_write", "head counts and block_size must be positive");
    if (head_dim % 8 == 0 && (((uintptr_t)qkv | (uintptr_t)cos_sin | (uintptr_t)q_out | (uintptr_t)k_cache |
                               (uintptr_t)v_cache) & 15) == 0)
        return launch_pdl("skv_rope_kv_write", rope_kv_write_vec_kernel<skv_t>, dim3((n_tokens + 3) / 4), dim3(128), 0, stream,
                          qkv, (const float2*)cos_sin, positions, token_seq, block_table, table_width, (skv_t*)q_out,
                          (skv_t*)k_cache, (skv_t*)v_cache, num_heads, num_kv_heads, head_dim, block_size, write_kv,
                          n_tokens);
    return launch_pdl("skv_rope_kv_write", rope_kv_write_kernel<skv_t>, dim3(n_tokens), dim3(128), 0, stream, qkv,
                      (const float2*)cos_sin, positions, token_seq, block_table, table_width, (skv_t*)q_out,
                      (skv_t*)k_cache, (skv_t*)v_cache, num_heads, num_kv_heads, head_dim, block_size, write_kv);
}

SKV_EXPORT int skv_add_inplace(float* out, const float* in, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    add_inplace_kernel<<<(int)blocks, threads, 0, stream>>>(out, in, (size_t)n);
    return check_launch("skv_add_inplace");
}
