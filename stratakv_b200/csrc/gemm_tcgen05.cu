// Prefill GEMM on the 5th-generation tensor cores: out = A[M,K] . W[N,K]^T, bfloat16 in,
// float accumulation in tensor memory, fused epilogue (the modes of linear.cu).
//
// This is what replaces the reference's 32x32 shared-memory tile GEMM
// (src/cuda/gemm_cuda.cu:445-525) when a step brings many tokens.  One block computes a
// 128 x BN tile of the output:
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor) of 128x64 A and BNx64 W tiles
//            into a ring of shared-memory stages, 128-byte swizzled, completing on mbarriers;
//   warp 1   allocates BN columns of tensor memory; one thread issues tcgen05.mma
//            (128 x BN x 16 per instruction, four per stage) and commits each stage back to
//            the loader, and the finished accumulator to the epilogue;
//   warps 2-5 read the accumulator with tcgen05.ld (each warp its quarter of the 128 lanes,
//            one output row per thread) and apply the epilogue.
// Tails in M, N and K are zero-filled by TMA and masked in the epilogue.
//
// Every wait on an mbarrier gives up after a bounded number of tries, raises bit 2 (value 4)
// of the caller's flag word, and lets the block drain and free its tensor memory.
#include "common.cuh"

#if SKV_DTYPE == SKV_BF16

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace skv {

enum { TC_MODE_STORE = 0, TC_MODE_STORE_F32 = 1, TC_MODE_ADD_F32 = 2, TC_MODE_GATED = 3 };

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;                      // 64 bfloat16 = one 128-byte swizzle row
constexpr int TC_THREADS = 192;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// Returns false if the barrier did not flip within the limit (the flag is raised then).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* flag) {
    for (uint32_t tries = 0; tries < TC_WAIT_LIMIT; ++tries) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    if (flag) atomicOr(flag, 4);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled:
// start address / 16 in bits 0-13, leading offset (unused here) 1 in bits 16-29, 1024 bytes
// between 8-row groups / 16 in bits 32-45, descriptor version 1 in bits 46-47, swizzle mode 2
// (128 bytes) in bits 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: D float (1 at bit 4), A and B bfloat16 (1 at bits 7 and
// 10), both K-major (bits 15, 16 zero), N/8 at bits 17-22, M/16 at bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ float silu_gate(float g) {
    const float sig = g >= 0.0f ? 1.0f / (1.0f + expf(-g)) : expf(g) / (1.0f + expf(g));
    return g * sig;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ out, int M, int N, int K, int mode, int* __restrict__ flag) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + (size_t)STAGES * STAGE_BYTES);     // full[STAGES], empty[STAGES], accum
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * BN;
    const int k_iters = (K + TC_BK - 1) / TC_BK;
    const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES), accum = smem_addr(bars + 2 * STAGES);

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                   // A is the previous kernel's output

    if (warp == 0 && lane == 0) {
        // ---- loader -------------------------------------------------------------------------
        bool ok = true;
        int armed = 0;
        for (int i = 0; i < k_iters && ok; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES) ok = mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, flag);
            if (!ok) break;
            const uint32_t a_dst = smem_addr(tiles + (size_t)s * STAGE_BYTES);
            mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
            tma_load_2d(a_dst, &map_a, i * TC_BK, m0, full0 + 8 * s);
            tma_load_2d(a_dst + A_BYTES, &map_w, i * TC_BK, n0, full0 + 8 * s);
            armed = i + 1;
        }
        if (!ok) {
            // let the copies in flight land before the block leaves (bounded)
            for (int i = max(0, armed - STAGES); i < armed; ++i) mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, nullptr);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- tensor-core issue ------------------------------------------------------------------
        constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
        bool ok = true;
        for (int i = 0; i < k_iters && ok; ++i) {
            const int s = i % STAGES;
            ok = mbar_wait(full0 + 8 * s, (i / STAGES) & 1, flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_addr(tiles + (size_t)s * STAGE_BYTES);
            const uint64_t a_desc = umma_desc(a_addr), w_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) {
                // 16 bfloat16 = 32 bytes further along K: +2 in the descriptor's 16-byte units
                umma_bf16(tmem_base, a_desc + 2 * k, w_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(empty0 + 8 * s);          // frees the stage when these MMAs have read it
        }
        umma_commit(accum);                       // arrives when every MMA above has finished
    } else if (warp >= 2) {
        // ---- epilogue ---------------------------------------------------------------------------
        const bool ok = mbar_wait(accum, 0, flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quarter = warp & 3;             // the TMEM lanes this warp may read
        const int m = m0 + quarter * 32 + lane;
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                tmem_load_32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (m >= M) continue;
                const int n = n0 + c;
                if (mode == TC_MODE_GATED) {
                    // columns come in groups of 16: 8 gate columns, then their 8 up columns
                    const int half_n = N >> 1;
                    __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)m * half_n + (n >> 1);
#pragma unroll
                    for (int grp = 0; grp < 2; ++grp) {
                        if (n + 16 * grp >= N) break;
                        __align__(16) __nv_bfloat16 r[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            r[j] = __float2bfloat16_rn(silu_gate(__uint_as_float(v[16 * grp + j])) *
                                                       __uint_as_float(v[16 * grp + 8 + j]));
                        *(uint4*)(dst + 8 * grp) = *(const uint4*)r;
                    }
                } else if (mode == TC_MODE_STORE) {
                    __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)m * N + n;
                    if (n + 32 <= N && (N & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            __align__(16) __nv_bfloat16 r[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) r[e] = __float2bfloat16_rn(__uint_as_float(v[j + e]));
                            *(uint4*)(dst + j) = *(const uint4*)r;
                        }
                    } else {
                        for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
                    }
                } else {
                    float* dst = (float*)out + (size_t)m * N + n;
                    const bool add = mode == TC_MODE_ADD_F32;
                    if (n + 32 <= N && (N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 r = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                   __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                            if (add) {
                                const float4 old = *(const float4*)(dst + j);
                                r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
                            }
                            *(float4*)(dst + j) = r;
                        }
                    } else {
                        for (int j = 0; j < 32 && n + j < N; ++j)
                            dst[j] = (add ? dst[j] : 0.0f) + __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return (EncodeTiled)entry;
    }();
    return fn;
}

struct MapKey {
    const void* base; int rows, cols, box_rows;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 0x9E3779B97F4A7C15ull) ^ ((size_t)k.cols << 21) ^ (size_t)k.box_rows;
    }
};

// A row-major [rows, cols] bfloat16 matrix, box of box_rows x 64 elements, 128-byte swizzle.
static int tensor_map(const void* base, int rows, int cols, int box_rows, CUtensorMap* out) {
    static std::mutex lock;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, rows, cols, box_rows};
    std::lock_guard<std::mutex> guard(lock);
    auto found = cache.find(key);
    if (found != cache.end()) { *out = found->second; return 0; }
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail("skv_linear(tcgen05)", "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap map;
    const CUresult status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                   elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) {
        char detail[64];
        snprintf(detail, sizeof detail, "cuTensorMapEncodeTiled failed with code %d", (int)status);
        return fail("skv_linear(tcgen05)", detail);
    }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return 0;
}

template <int BN, int STAGES>
static int launch_tc(const void* a, const void* w, void* out, int M, int N, int K, int mode, int* flag,
                     cudaStream_t stream) {
    CUtensorMap map_a, map_w;
    if (int code = tensor_map(a, M, K, TC_BM, &map_a)) return code;
    if (int code = tensor_map(w, N, K, BN, &map_w)) return code;
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        const cudaError_t status = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skv_linear(tcgen05)", cudaGetErrorString(status));
        configured = true;
    }
    dim3 grid((M + TC_BM - 1) / TC_BM, (N + BN - 1) / BN);
    return launch_pdl("skv_linear(tcgen05)", gemm_tcgen05_kernel<BN, STAGES>, grid, dim3(TC_THREADS), smem, stream,
                      map_a, map_w, out, M, N, K, mode, flag);
}

int linear_tcgen05(const void* a, const void* w, void* out, int M, int N, int K, int mode, int* flag,
                   cudaStream_t stream) {
    if (K % 8 != 0) return fail("skv_linear(tcgen05)", "the inner size must be a multiple of 8 (16-byte rows)");
    if (((uintptr_t)a | (uintptr_t)w) & 15) return fail("skv_linear(tcgen05)", "operands must be 16-byte aligned");
    if (mode == TC_MODE_GATED && N % 16 != 0) return fail("skv_linear(tcgen05)", "a gated weight needs a multiple of 16 rows");
    return launch_tc<128, 4>(a, w, out, M, N, K, mode, flag, stream);
}

}  // namespace skv

#endif
