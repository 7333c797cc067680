// Linear layers: out = A[M,K] . W[N,K]^T with a fused epilogue.
//
// W keeps the checkpoint's [out, in] rows (K contiguous), as the reference's
// GPU path does (src/generation/generator.cpp:311-319).  These kernels replace
// its warp-per-output GEMV and 32x32 tile GEMM (src/cuda/gemm_cuda.cu:445-608)
// and the separate add and SwiGLU kernels that follow them (:221-231, 276-284).
//
// Epilogues (`mode`):
//   0 STORE      out[M,N] in the compute dtype
//   1 STORE_F32  out[M,N] float
//   2 ADD_F32    out[M,N] float += result          (residual sum in float)
//   3 GATED      W rows come in tiles of 16: rows 0-7 of a tile are gate rows
//                8t..8t+7, rows 8-15 the matching up rows; out[M,N/2] =
//                act(gate) * up in the compute dtype
//
// float build: a true 32-bit FMA tile kernel (no tensor cores, no TF32).
// bfloat16 build: a weight-streaming kernel for any M that keeps 16 weight rows
// per block and feeds tokens in groups of 8 through mma.sync m16n8k16 with float
// accumulation.  Each lane loads 16 bytes (8 consecutive k) of a weight row and of
// a token row and issues two MMAs on them; the k order inside an MMA is permuted
// the same way for both operands, which leaves the dot products unchanged.
#include "common.cuh"

namespace skv {

enum { MODE_STORE = 0, MODE_STORE_F32 = 1, MODE_ADD_F32 = 2, MODE_GATED = 3 };

__device__ __forceinline__ float activate(float g, int act) {
    if (act == ACT_GELU_TANH) return gelu_tanh(g);
    // silu(g) = g * sigmoid(g); the two-branch sigmoid of the reference's CPU
    // block (src/models/transformer_block.cpp:315-323) avoids overflow of exp.
    const float sig = g >= 0.0f ? 1.0f / (1.0f + expf(-g)) : expf(g) / (1.0f + expf(g));
    return g * sig;
}

template <typename T>
__device__ __forceinline__ void epilogue_store(void* out, int mode, int M, int N, int m, int n, float v) {
    if (m >= M || n >= N) return;
    const size_t at = (size_t)m * N + n;
    if (mode == MODE_STORE) ((T*)out)[at] = from_float<T>(v);
    else if (mode == MODE_STORE_F32) ((float*)out)[at] = v;
    else ((float*)out)[at] += v;
}

#if SKV_DTYPE == SKV_F32
// ---------------------------------------------------------------------------
// 64x64 output tile, K in steps of 16, 256 threads, 4 tokens x 4 columns each.
// A thread's columns are {2j, 2j+1, 2j+8, 2j+9} of one 16-column group so that a
// gate column and its up column meet in one thread.
constexpr int FBM = 64, FBN = 64, FBK = 16;

__global__ void __launch_bounds__(256)
linear_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, void* __restrict__ out,
                  int M, int N, int K, int mode, int act) {
    __shared__ float As[FBK][FBM + 4];
    __shared__ float Ws[FBK][FBN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * FBM, n0 = blockIdx.x * FBN;
    const int group = tx >> 2, j = tx & 3;
    int cols[4] = {16 * group + 2 * j, 16 * group + 2 * j + 1, 16 * group + 2 * j + 8, 16 * group + 2 * j + 9};
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += FBK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int row = e >> 4, k = e & 15;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + k;
            As[k][row] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.0f;
            Ws[k][row] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < FBK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int c = 0; c < 4; ++c) w[c] = Ws[k][cols[c]];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[i][c] = fmaf(a[i], w[c], acc[i][c]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (mode == MODE_GATED) {
            if (m >= M) continue;
            const int half_n = N >> 1;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int n = n0 + cols[c];            // a gate row of W; its up row is n + 8
                if (n >= N) continue;
                const int o = ((n >> 4) << 3) + (n & 7);
                if (o < half_n)
                    ((float*)out)[(size_t)m * half_n + o] = activate(acc[i][c], act) * acc[i][c + 2];
            }
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) epilogue_store<float>(out, mode, M, N, m, n0 + cols[c], acc[i][c]);
        }
    }
}

struct NormArgs { const float* row_scale; const float* partials_in; int n_partials_in, stride_in; float eps_in;
                  const int* rows; float* partials; int partial_stride; unsigned int* counter;
                  const float* gamma_next; float eps_next; void* scaled_out; float* row_scale_out; };

static int launch_linear(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act,
                         int* flag, const NormArgs& norm, cudaStream_t stream) {
    (void)flag;
    if (norm.row_scale || norm.partials_in || norm.partials) return fail("skv_linear(float)", "the norm-fused form exists in the bfloat16 build only");
    dim3 grid((N + FBN - 1) / FBN, (M + FBM - 1) / FBM);
    return launch_pdl("skv_linear(float)", linear_f32_kernel, grid, dim3(256), 0, stream, (const float*)a,
                      (const float*)w, out, M, N, K, mode, act);
}

#else  // bfloat16
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool STREAM>
__device__ __forceinline__ uint4 load_weight16(const uint4* p) {
    return STREAM ? __ldcs(p) : __ldg(p);
}

// RMSNorm folded into the projections around it.  The kernel that updates the float residual stream
// (residual-add mode) also leaves, per token, the updated row times the NEXT norm's weight in bfloat16
// and the factor 1 / sqrt(mean(row^2) + eps); the projection after that norm takes those activations
// and multiplies its result by the factor, which is one number per token and so commutes with the
// product.  Everything about the norm stays in float; the activations are rounded to bfloat16 once, as
// they are when the norm runs as a kernel of its own.
// A row's sum of squares is made in a fixed order whatever the timing: every block of the producer leaves
// the sum over its 16 columns.  With few tokens the consumer adds them up itself: it copies the partial sums
// of its tokens to shared memory while its main loop runs, so the producer ends without further ado.  With
// many tokens that would be a lot of traffic for every consumer block, and the producer's block that
// finishes last (a counter tells it) adds them up once and leaves the factor.
struct NormArgs {
    // consumer side: the factor itself, or the partial sums to make it from (both null: plain projection)
    const float* row_scale;        // [rows] factor of each row of X
    const float* partials_in;      // [rows, stride_in]: n_partials_in partial sums of squares per row
    int n_partials_in, stride_in;
    float eps_in;
    const int* rows;               // token m reads row rows[m] of X and of the above (null: row m)
    // producer side, residual-add mode (null partials: not wanted)
    float* partials;               // [M, partial_stride], partial_stride >= blocks of the grid
    int partial_stride;
    const float* gamma_next;       // [N] weight of the norm that reads the stream next
    __nv_bfloat16* scaled_out;     // [M, N] = bfloat16(updated out * gamma_next)
    unsigned int* counter;         // null: the consumer sums the partials; else zero before the launch and after it
    float eps_next;
    float* row_scale_out;          // with counter: [M] = 1 / sqrt(mean(updated out[m, :]^2) + eps_next)
};

// One block owns 16 rows of W and one chunk of 8*TG tokens.  Its warps take the
// 32-wide k steps round robin, then their partial tiles are summed in shared
// memory in warp order (a fixed order: results do not depend on timing).
// Weights do not depend on the kernel before this one, so the first batch of
// weight loads is issued before pdl_wait(): it overlaps the predecessor's tail.
template <int TG, int U, bool STREAM, int MAX_WARPS>
__global__ void __launch_bounds__(MAX_WARPS * 32, MAX_WARPS == 4 ? (TG == 1 ? 5 : (TG == 2 ? 5 : 2)) : (MAX_WARPS == 8 && TG <= 2 ? 2 : 1))
skinny_linear_bf16_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                          void* __restrict__ out, int M, int N, int K, int mode, int act, const NormArgs norm) {
    extern __shared__ float red[];                 // [warps][16][8*TG + 1], [8*TG] factors, [8*TG][n_partials_in] partial sums
    constexpr int COLS = 8 * TG, PITCH = COLS + 1;
    pdl_launch_dependents();
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int n0 = blockIdx.x * 16, m0 = blockIdx.y * COLS;
    const int steps = (K + 31) >> 5;

    const int row_a = min(n0 + g, N - 1), row_b = min(n0 + g + 8, N - 1);
    const bool has_a = n0 + g < N, has_b = n0 + g + 8 < N;
    const __nv_bfloat16* wa_ptr = W + (size_t)row_a * K + tig * 8;
    const __nv_bfloat16* wb_ptr = W + (size_t)row_b * K + tig * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    uint4 wa[U], wb[U];
    auto load_weights = [&](int s0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (s0 + u * warps) << 5;
            const bool live = (s0 + u * warps) < steps && (k + tig * 8) < K;
            wa[u] = (live && has_a) ? load_weight16<STREAM>((const uint4*)(wa_ptr + k)) : zero;
            wb[u] = (live && has_b) ? load_weight16<STREAM>((const uint4*)(wb_ptr + k)) : zero;
        }
    };
    load_weights(warp);
    pdl_wait();                                    // activations (and the residual stream) are ready now

    const __nv_bfloat16* x_ptr[TG];
    bool has_x[TG];
#pragma unroll
    for (int t = 0; t < TG; ++t) {
        const int m = m0 + t * 8 + g;
        has_x[t] = m < M;
        const int safe = min(m, M - 1);
        x_ptr[t] = X + (size_t)(norm.rows ? norm.rows[safe] : safe) * K + tig * 8;
    }
    float* factor = red + (size_t)warps * 16 * PITCH;
    float* staged = factor + COLS;
    if (norm.partials_in) {
        // the partial sums are wanted after the main loop: they travel to shared memory meanwhile, 16 bytes
        // at a time where the rows allow it (the row in shared memory is `pitch` floats)
        const bool wide = (norm.stride_in & 3) == 0 && ((uintptr_t)norm.partials_in & 15) == 0;
        const int pitch = (norm.n_partials_in + 3) & ~3;
        const int pieces = wide ? pitch >> 2 : norm.n_partials_in;
        for (int i = threadIdx.x; i < COLS * pieces; i += blockDim.x) {
            const int m = i / pieces, piece = i - m * pieces;
            if (m0 + m < M) {
                const float* row = norm.partials_in + (size_t)(norm.rows ? norm.rows[m0 + m] : m0 + m) * norm.stride_in;
                if (wide)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(staged + m * pitch + 4 * piece)),
                                 "l"(row + 4 * piece) : "memory");
                else
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(staged + m * pitch + piece)),
                                 "l"(row + piece) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    } else if (norm.row_scale && !norm.rows && threadIdx.x * 32 < M) {
        // the factors are wanted after the main loop: bring their lines close meanwhile
        asm volatile("prefetch.global.L1 [%0];" ::"l"(norm.row_scale + threadIdx.x * 32));
    }
    float acc[TG][4];
#pragma unroll
    for (int t = 0; t < TG; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f; }

    for (int s0 = warp; s0 < steps; s0 += warps * U) {
        if (s0 != warp) load_weights(s0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (s0 + u * warps) << 5;
            const bool live = (s0 + u * warps) < steps && (k + tig * 8) < K;
#pragma unroll
            for (int t = 0; t < TG; ++t) {
                const uint4 xv = (live && has_x[t]) ? *(const uint4*)(x_ptr[t] + k) : zero;
                mma_bf16_16816(acc[t], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
                mma_bf16_16816(acc[t], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
            }
        }
    }
    if (norm.partials_in) {
        asm volatile("cp.async.wait_all;\n" ::: "memory");
        __syncthreads();
        for (int m = warp; m < COLS; m += warps) {          // one token per warp at a time, lanes in a fixed order
            float total = 0.0f;
            const int pitch = (norm.n_partials_in + 3) & ~3;
            for (int p = lane; p < norm.n_partials_in; p += 32) total += staged[m * pitch + p];
            total = warp_sum(total);
            if (lane == 0) factor[m] = 1.0f / sqrtf(total / (float)K + norm.eps_in);
        }
    }
    float* mine = red + (size_t)warp * 16 * PITCH;
#pragma unroll
    for (int t = 0; t < TG; ++t) {
        mine[g * PITCH + t * 8 + 2 * tig] = acc[t][0];
        mine[g * PITCH + t * 8 + 2 * tig + 1] = acc[t][1];
        mine[(g + 8) * PITCH + t * 8 + 2 * tig] = acc[t][2];
        mine[(g + 8) * PITCH + t * 8 + 2 * tig + 1] = acc[t][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * COLS; idx += blockDim.x) {
        const int r = idx & 15, m = idx >> 4;
        float sum = 0.0f;
        for (int w = 0; w < warps; ++w) sum += red[((size_t)w * 16 + r) * PITCH + m];
        if (norm.partials_in) sum *= factor[m];
        else if (norm.row_scale && m0 + m < M) sum *= norm.row_scale[norm.rows ? norm.rows[m0 + m] : m0 + m];
        red[(size_t)r * PITCH + m] = sum;          // warp 0's tile becomes the total
        // (each (r, m) is read and written by this thread only)
    }
    __syncthreads();
    if (mode == MODE_GATED) {
        const int half_n = N >> 1;
        for (int idx = threadIdx.x; idx < 8 * COLS; idx += blockDim.x) {
            const int r = idx & 7, m = idx >> 3;
            const int o = (n0 >> 1) + r, gm = m0 + m;
            if (gm < M && o < half_n) {
                const float gate = red[(size_t)r * PITCH + m], up = red[(size_t)(r + 8) * PITCH + m];
                ((__nv_bfloat16*)out)[(size_t)gm * half_n + o] = __float2bfloat16_rn(activate(gate, act) * up);
            }
        }
    } else if (mode == MODE_ADD_F32 && norm.partials) {
        // residual sum; the updated row times the next norm's weight; its sum of squares over this block's columns
        for (int idx = threadIdx.x; idx < 16 * COLS; idx += blockDim.x) {        // whole warps stay together
            const int r = idx & 15, m = idx >> 4;
            float updated = 0.0f;
            if (m0 + m < M && n0 + r < N) {
                float* at = (float*)out + (size_t)(m0 + m) * N + n0 + r;
                updated = *at + red[(size_t)r * PITCH + m];
                *at = updated;
                norm.scaled_out[(size_t)(m0 + m) * N + n0 + r] = __float2bfloat16_rn(updated * norm.gamma_next[n0 + r]);
            }
            float square = updated * updated;
#pragma unroll
            for (int offset = 8; offset > 0; offset >>= 1) square += __shfl_xor_sync(0xffffffffu, square, offset);
            if (r == 0 && m0 + m < M) norm.partials[(size_t)(m0 + m) * norm.partial_stride + blockIdx.x] = square;
        }
        if (!norm.counter) return;                  // the consumer adds the partial sums up
        // the last block to get here adds them up (the grid has one chunk of tokens: M <= 8*TG)
        __shared__ bool last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) last = atomicAdd(norm.counter, 1u) == gridDim.x - 1;
        __syncthreads();
        if (last) {
            __threadfence();
            for (int m = warp; m < M; m += warps) {
                const float* partial = norm.partials + (size_t)m * norm.partial_stride;
                float total = 0.0f;
                for (int p = lane; p < (int)gridDim.x; p += 32) total += __ldcg(partial + p);
                total = warp_sum(total);
                if (lane == 0) norm.row_scale_out[m] = 1.0f / sqrtf(total / (float)N + norm.eps_next);
            }
            if (threadIdx.x == 0) *norm.counter = 0u;
        }
    } else {
        for (int idx = threadIdx.x; idx < 16 * COLS; idx += blockDim.x) {
            const int r = idx & 15, m = idx >> 4;
            epilogue_store<__nv_bfloat16>(out, mode, M, N, m0 + m, n0 + r, red[(size_t)r * PITCH + m]);
        }
    }
}

template <int TG, int U, int MAX_WARPS>
static int launch_skinny_as(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act,
                            int warps, const NormArgs& norm, cudaStream_t stream) {
    const int row_tiles = (N + 15) / 16, chunks = (M + 8 * TG - 1) / (8 * TG);
    const size_t smem = ((size_t)warps * 16 * (8 * TG + 1) + 8 * TG + (size_t)8 * TG * (norm.partials_in ? (norm.n_partials_in + 3) & ~3 : 0)) * sizeof(float);
    if (smem > 48 * 1024) return fail("skv_linear(bfloat16)", "too many partial sums for the consumer to stage: let the producer finish them");
    dim3 grid(row_tiles, chunks);
    if (chunks == 1)
        return launch_pdl("skv_linear(bfloat16)", skinny_linear_bf16_kernel<TG, U, true, MAX_WARPS>, grid,
                          dim3(warps * 32), smem, stream, (const __nv_bfloat16*)w, (const __nv_bfloat16*)a, out, M, N,
                          K, mode, act, norm);
    return launch_pdl("skv_linear(bfloat16)", skinny_linear_bf16_kernel<TG, U, false, MAX_WARPS>, grid,
                      dim3(warps * 32), smem, stream, (const __nv_bfloat16*)w, (const __nv_bfloat16*)a, out, M, N, K,
                      mode, act, norm);
}

// Warps per block.  Four to five row tiles per SM: 4 warps, compiled to fit 5 blocks on an SM so that
// e.g. 704 tiles run as one wave.  Fewer row tiles, or more than one such wave holds: 8 warps (two blocks fit on an
// SM, so the next kernel's weight loads overlap this one's end; with many tiles, blocks of 8 warps that come and go
// keep the memory pipe fuller than two waves of 4-warp blocks: 22,016 x 4,096 at 8 tokens 44.2 -> 35.9 us, 32,000 x
// 2,048 31.6 -> 28.3 us), or 16 when the inner size is so long that 8 warps would need more than two rounds of loads
// each and the tiles are no more than the SMs (a block of 16 warps has an SM to itself; 256 tiles of 8 warps run as
// one wave, of 16 warps as two).  Never more warps than k steps.
template <int TG, int U, int MAX_WARPS>
static int launch_skinny(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act,
                         const NormArgs& norm, cudaStream_t stream) {
    const int row_tiles = (N + 15) / 16, chunks = (M + 8 * TG - 1) / (8 * TG);
    const int steps = (K + 31) / 32;
    const long long blocks = (long long)row_tiles * chunks;
    const int sms = sm_count();
    int warps = (blocks >= sms * 4 && blocks <= sms * 5) ? 4 : 8;
    // (Blocks of 3 warps, of which 7 fit on an SM, were once used for a few more tiles than five blocks of 4 warps per SM
    // hold, 768 at hidden size 4096; blocks of 8 warps measured faster there too: 12,288 x 4,096 at 8 tokens 27.9 -> 22.5 us.)
    if (warps == 8 && MAX_WARPS >= 16 && steps > 8 * U * 2 && blocks <= sms) warps = 16;   // (16 warps: one block per SM)
    if (warps > MAX_WARPS) warps = MAX_WARPS;
    while (warps > 1 && warps > steps) warps >>= 1;
    if (warps <= 4) return launch_skinny_as<TG, U, 4>(a, w, out, M, N, K, mode, act, warps, norm, stream);
    if (warps <= 8 || MAX_WARPS < 16) return launch_skinny_as<TG, U, 8>(a, w, out, M, N, K, mode, act, warps, norm, stream);
    return launch_skinny_as<TG, U, 16>(a, w, out, M, N, K, mode, act, warps, norm, stream);
}

// gemm_tcgen05.cu: the tensor-memory GEMM that serves steps with many tokens
int linear_tcgen05(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act, int* flag,
                   cudaStream_t stream);

static int launch_linear(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act,
                         int* flag, const NormArgs& norm, cudaStream_t stream) {
    if (K % 8 != 0)
        return fail("skv_linear(bfloat16)", "the inner size must be a multiple of 8 (16-byte rows)");
    if (((uintptr_t)a | (uintptr_t)w) & 15)
        return fail("skv_linear(bfloat16)", "operands must be 16-byte aligned");
    if ((norm.row_scale || norm.partials_in || norm.partials) && M > 64)
        return fail("skv_linear(bfloat16)", "the norm-fused form serves steps of at most 64 tokens");
    // above 16 tokens the tensor-memory kernels take over, unless a norm is folded into this projection
    if (M > 16 && !norm.row_scale && !norm.partials_in && !norm.partials)
        return linear_tcgen05(a, w, out, M, N, K, mode, act, flag, stream);
    // at most 8 warps and under 100 registers a thread: two blocks fit on an SM, so the next
    // kernel's weight loads are in flight while this one finishes
    if (M <= 8) return launch_skinny<1, 8, 16>(a, w, out, M, N, K, mode, act, norm, stream);
    if (M <= 16) return launch_skinny<2, 8, 16>(a, w, out, M, N, K, mode, act, norm, stream);
    if (M <= 32) return launch_skinny<4, 4, 8>(a, w, out, M, N, K, mode, act, norm, stream);
    return launch_skinny<8, 4, 8>(a, w, out, M, N, K, mode, act, norm, stream);
}
#endif

}  // namespace skv

using namespace skv;

static int check_linear(int M, int N, int K, int mode, int act) {
    if (N <= 0 || K <= 0) return fail("skv_linear", "N and K must be positive");
    if (mode < 0 || mode > 3) return fail("skv_linear", "unknown epilogue mode");
    if (mode == MODE_GATED && N % 16 != 0)
        return fail("skv_linear", "a gated weight must have a multiple of 16 rows (gate/up tiles of 8)");
    if (act < 0 || act >= ACT_COUNT) return fail("skv_linear", "unknown activation");
    (void)M;
    return 0;
}

// `flag` (may be null): bit 2 (value 4) is raised if a pipeline wait inside a kernel timed out.
// With `scaled_out` (residual-add mode, at most 64 tokens, bfloat16 build) the kernel also leaves what the
// projection after the next norm needs (see NormArgs): the scaled rows, and the rows' sums of squares as
// `partials` [M, partial_stride] with partial_stride >= N/16 rounded up.  With `counter` (one zeroed word, left
// zeroed) it finishes them into `row_scale_out` too.
SKV_EXPORT int skv_linear(const void* a, const void* w, void* out, int M, int N, int K, int mode, int act,
                          int* flag, void* scaled_out, const float* gamma_next, float* partials, int partial_stride,
                          float* row_scale_out, float eps_next, unsigned int* counter, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (int code = check_linear(M, N, K, mode, act)) return code;
    NormArgs norm = {};
    if (scaled_out) {
        if (mode != MODE_ADD_F32) return fail("skv_linear", "a norm is folded into the residual-add mode only");
        if (!gamma_next || !partials || partial_stride < (N + 15) / 16 || (counter && !row_scale_out))
            return fail("skv_linear", "the next norm's weight, room for N/16 partial sums per token and, with a counter, a place for the factors are needed");
        norm.partials = partials;
        norm.partial_stride = partial_stride;
        norm.gamma_next = gamma_next;
        norm.scaled_out = (decltype(norm.scaled_out))scaled_out;
        norm.counter = counter;
        norm.eps_next = eps_next;
        norm.row_scale_out = row_scale_out;
    }
    return launch_linear(a, w, out, M, N, K, mode, act, flag, norm, stream);
}

// The projection after a folded norm: `a` holds rows of (stream * norm weight) in bfloat16, token m reads
// row rows[m] (or m), and the result is multiplied by the row's factor: row_scale[row], or (row_scale null)
// 1 / sqrt(sum of partials[row, :n_partials] / K + eps).  bfloat16 build, at most 64 tokens.
SKV_EXPORT int skv_linear_normed(const void* a, const float* row_scale, const float* partials, int n_partials,
                                 int partial_stride, float eps, const int* rows, const void* w, void* out, int M,
                                 int N, int K, int mode, int act, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (int code = check_linear(M, N, K, mode, act)) return code;
    if (!row_scale && (!partials || n_partials <= 0 || partial_stride < n_partials))
        return fail("skv_linear_normed", "the rows' factors, or their partial sums of squares, are needed");
    NormArgs norm = {};
    if (row_scale) {
        norm.row_scale = row_scale;
    } else {
        norm.partials_in = partials;
        norm.n_partials_in = n_partials;
        norm.stride_in = partial_stride;
        norm.eps_in = eps;
    }
    norm.rows = rows;
    return launch_linear(a, w, out, M, N, K, mode, act, nullptr, norm, stream);
}
