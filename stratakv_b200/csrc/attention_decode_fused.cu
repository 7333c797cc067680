// Decode attention with its neighbours folded in (bfloat16): rotary encoding of the new
// token's queries and key, the write of that key and value into the paged cache, the
// split-KV attention itself, and the merge of the splits, as one kernel.
//
// It replaces four launches of the unfused path (rope_kv_write_kernel, decode_attention_kernel,
// decode_combine_kernel; in the reference: generate_rope_frequencies, rope_split_half x2, two
// cache-append copies and paged_attention_decode_kernel, src/models/transformer_block.cpp:
// 457-518).  The arithmetic is the same as in elementwise.cu and attention_decode.cu: pairs
// (i, i + head_dim/2) rotate in float with a host-built cos/sin table, queries and keys are
// rounded to bfloat16 once, scores / softmax / output accumulate in float.
//
// The kernel is built around its latency chain, since a decode step gives it little else to
// win: at batch 8 and 2,048 keys a block reads 64 KB.
//  * Keys and values of earlier positions cannot change during the step, so a block starts
//    streaming its piece of the context into shared memory (cp.async, two stages of 128 keys)
//    as soon as it is resident, before it waits for the q|k|v projection in front of it.
//  * After the wait one round of 16-byte loads fetches the queries (and the new key and value in
//    the block that owns the newest position); they are rotated into a shared tile, the new row
//    goes to the cache and straight into the staged keys.  Fragments come from ldmatrix.
//  * The splits of one (sequence, KV head) are the blocks of a thread-block cluster.  Each block
//    pushes its partial (max, sum, output) rows into the shared memory of the block that owns the
//    row, one cluster barrier makes them visible, and the owner merges and writes the row.  No
//    scratch in global memory, no second kernel, no barrier after the merge.
#include "common.cuh"


// Two stages of 128 keys and values must fit one block's shared memory, which holds for head sizes up
// to 192; above that this kernel is not built and the separate kernels (elementwise.cu,
// attention_decode.cu) serve, as skv_has_attention_decode_fused() tells the caller.
#if SKV_DTYPE == SKV_BF16 && SKV_HEAD_DIM <= 192

namespace skv {

constexpr int FHD = SKV_HEAD_DIM;
constexpr int FKSTEPS = FHD / 16, FOTILES = FHD / 8;
constexpr int FWARPS = 8, FTHREADS = FWARPS * 32;
constexpr int FCHUNK = FWARPS * 16;                 // keys per stage: one group of 16 per warp
constexpr int FMAX_STAGES = 4;                      // stages per launch: 2 .. FMAX_STAGES (see the launch below)
// Staged rows: ldmatrix reads 16 bytes of each of 8 neighbouring rows at once, which must fall on different banks.
// Rows of whole 128-byte multiples are stored with their 16-byte pieces exchanged (piece ^ (row & 7)), at no cost
// in space; other head sizes get 16 bytes of padding per row.
constexpr bool FSWIZZLED = (FHD * 2) % 128 == 0;
constexpr int FROW = FSWIZZLED ? FHD * 2 : FHD * 2 + 16;
constexpr int FQROW = FHD * 2 + 16;                 // bytes between rows of the query tile and the new rows (padded)
__device__ __forceinline__ uint32_t f_staged(int row, int piece) {          // byte offset of a row's 16-byte piece in a stage
    return (uint32_t)(row * FROW + ((FSWIZZLED ? piece ^ (row & 7) : piece) << 4));
}
constexpr int FPIECES = FHD / 8;                    // 16-byte pieces per row
constexpr int FSTAGE_BYTES = 2 * FCHUNK * FROW;     // keys, then values
constexpr int FPITCH = FHD + 2;                     // floats per partial row: outputs, max, sum
constexpr int FINBOX_ROWS = 24;                     // >= ceil(16 / blocks) * blocks for 1..8 blocks

// shared memory, in bytes from the start
constexpr int F_Q_AT = 0;                                           // [16][FQROW] rotated queries
constexpr int F_NEW_AT = F_Q_AT + 16 * FQROW;                       // new key row, new value row
constexpr int F_ANGLES_AT = F_NEW_AT + 2 * FQROW;                   // [FHD/2] (cos, sin)
constexpr int F_INBOX_AT = F_ANGLES_AT + (FHD / 2) * 8;             // [FINBOX_ROWS][FPITCH] floats, written by the cluster
constexpr int FTABLE = 512;                                         // entries of the block table kept in shared memory
constexpr int F_TABLE_AT = F_INBOX_AT + FINBOX_ROWS * FPITCH * 4;   // [FTABLE] ints
constexpr int F_STAGES_AT = (F_TABLE_AT + FTABLE * 4 + 127) / 128 * 128;   // also the warps' merge area after the loop
constexpr int F_SMEM_LIMIT = 227 * 1024;
static_assert(FWARPS * 16 * FPITCH * 4 <= 2 * FSTAGE_BYTES, "the merge area reuses the stages");
static_assert(F_STAGES_AT + 2 * FSTAGE_BYTES <= F_SMEM_LIMIT, "shared memory");

__device__ __forceinline__ void f_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void f_ldmatrix(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

__device__ __forceinline__ void f_ldmatrix_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}

// 16 bytes global -> shared, asynchronously; `bytes` 0 writes zeros instead
__device__ __forceinline__ void f_copy16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void f_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void f_wait_copies() { asm volatile("cp.async.wait_group %0;\n" ::"n"(PENDING) : "memory"); }

__device__ __forceinline__ void f_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void f_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t f_cluster_rank() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r)); return r;
}
__device__ __forceinline__ uint32_t f_cluster_size() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r)); return r;
}
// the address, in the cluster's shared window, of `local` (a shared address of this block) in block `rank`
__device__ __forceinline__ uint32_t f_remote(uint32_t local, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local), "r"(rank)); return r;
}
__device__ __forceinline__ void f_remote_store(uint32_t address, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(address), "f"(v) : "memory");
}

__device__ __forceinline__ float f_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t f_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&v;
}

__global__ void __launch_bounds__(FTHREADS, FHD <= 64 ? 2 : 1)
decode_attention_fused_kernel(const float* __restrict__ qkv, const float2* __restrict__ cos_sin,
                              __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                              const int* __restrict__ block_table, int table_width,
                              const int* __restrict__ ctx_after, __nv_bfloat16* __restrict__ out, int num_heads,
                              int num_kv_heads, int block_size, float scale, int window, int splits, int m_tiles,
                              int write_kv, int block_shift, int stages) {
    extern __shared__ __align__(128) unsigned char fused_smem[];
    constexpr int HALF = FHD / 2;
    pdl_launch_dependents();
    f_cluster_arrive();                               // "this block is running": waited for before the first remote store
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int seq = blockIdx.x;
    const int kv_head = blockIdx.y / m_tiles, m_tile = blockIdx.y - kv_head * m_tiles;
    const int split = blockIdx.z;
    const int group_size = num_heads / num_kv_heads;
    const int head0 = kv_head * group_size + m_tile * 16;
    const int rows = min(16, group_size - m_tile * 16);
    const int q_dim = num_heads * FHD, kv_dim = num_kv_heads * FHD;

    // The block table's row goes to shared memory while the context length is on its way, so that the
    // copies below start after one round trip to memory, not two.
    const int* table = block_table + (size_t)seq * table_width;
    int* table_near = (int*)(fused_smem + F_TABLE_AT);
    for (int i = threadIdx.x; i < min(table_width, FTABLE); i += FTHREADS) table_near[i] = table[i];
    const int ctx = ctx_after[seq];
    const int pos = ctx - 1;                          // the new token's position
    const int lo = window > 0 ? max(0, ctx - window) : 0;
    const int first_group = lo >> 4, end_group = (ctx + 15) >> 4;
    const int per_split = (end_group - first_group + splits - 1) / splits;
    const int my_first = first_group + split * per_split;
    const int my_end = min(end_group, my_first + per_split);
    const int n_chunks = my_end > my_first ? (my_end - my_first + FWARPS - 1) / FWARPS : 0;
    const float scale_log2 = scale * 1.4426950408889634f;
    const float* token = qkv + (size_t)seq * (q_dim + 2 * kv_dim);
    const int newest_group = pos >> 4;
    const bool owns_newest = newest_group >= my_first && newest_group < my_end;

    const uint32_t smem = smem_u32(fused_smem);
    float2* angles = (float2*)(fused_smem + F_ANGLES_AT);
    float* inbox = (float*)(fused_smem + F_INBOX_AT);
    // rotation angles of the new position come from a table that the step does not write
    static_assert(FHD / 2 <= FTHREADS, "one angle per thread");
    float2 my_angle = make_float2(1.0f, 0.0f);
    if (cos_sin && threadIdx.x < HALF) my_angle = cos_sin[(size_t)pos * HALF + threadIdx.x];
    __syncthreads();                                  // the table is in shared memory
    auto block_of = [&](int key) {
        const int index = block_shift >= 0 ? key >> block_shift : key / block_size;
        return index < FTABLE ? table_near[index] : table[index];
    };
    auto row_in_block = [&](int key) { return block_shift >= 0 ? key & (block_size - 1) : key % block_size; };

    // Stage chunk c (groups my_first + 8c ...) of this block's keys and values.  Rows past the context are
    // zero-filled: a masked key has weight 0, and 0 times whatever lay in shared memory need not be 0.
    auto issue_chunk = [&](int c) {
        if (c < n_chunks) {
            const int key0 = (my_first + c * FWARPS) << 4;
            const int key_end = min(ctx, my_end << 4);
            const uint32_t stage = smem + F_STAGES_AT + (c % stages) * FSTAGE_BYTES;
            for (int i = threadIdx.x; i < FCHUNK * FPIECES; i += FTHREADS) {
                const int row = i / FPIECES, piece = i - row * FPIECES;
                const int key = key0 + row;
                const bool live = key < key_end;
                size_t at = 0;
                if (live)
                    at = ((size_t)(block_of(key) * num_kv_heads + kv_head) * block_size + row_in_block(key)) * FHD + piece * 8;
                const uint32_t dst = stage + f_staged(row, piece);
                f_copy16(dst, k_cache + at, live ? 16 : 0);
                f_copy16(dst + FCHUNK * FROW, v_cache + at, live ? 16 : 0);
            }
        }
        f_commit();
    };
    // Keys and values of earlier positions were written by earlier steps (and the one row that this step
    // writes is replaced below), so the copies need not wait for the kernel in front.
    for (int c = 0; c < stages; ++c) issue_chunk(c);
    if (threadIdx.x < HALF) angles[threadIdx.x] = my_angle;
    // query rows that no head fills stay zero
    for (int i = threadIdx.x; i < 16 * FQROW / 16; i += FTHREADS)
        *(uint4*)(fused_smem + F_Q_AT + i * 16) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    pdl_wait();

    // Queries (and the new key, where this block owns the newest position and the layer writes its cache):
    // item `rows` is the key.  One thread rotates four pairs (d, d + HALF).
    {
        const bool with_key = owns_newest && write_kv;
        const int items = (rows + (with_key ? 1 : 0)) * (HALF / 4);
        size_t new_at = 0;
        if (owns_newest)
            new_at = ((size_t)(block_of(pos) * num_kv_heads + kv_head) * block_size + row_in_block(pos)) * FHD;
        for (int i = threadIdx.x; i < items; i += FTHREADS) {
            const int item = i / (HALF / 4), quad = i - item * (HALF / 4);
            const float* x = item < rows ? token + (size_t)(head0 + item) * FHD : token + q_dim + (size_t)kv_head * FHD;
            const float4 a = *(const float4*)(x + 4 * quad), b = *(const float4*)(x + HALF + 4 * quad);
            const float xa[4] = {a.x, a.y, a.z, a.w}, xb[4] = {b.x, b.y, b.z, b.w};
            float first[4], second[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 cs = angles[4 * quad + e];
                first[e] = xa[e] * cs.x - xb[e] * cs.y;          // as rotated() of elementwise.cu
                second[e] = xa[e] * cs.y + xb[e] * cs.x;
            }
            const uint2 low = make_uint2(f_pack(first[0], first[1]), f_pack(first[2], first[3]));
            const uint2 high = make_uint2(f_pack(second[0], second[1]), f_pack(second[2], second[3]));
            unsigned char* row = item < rows ? fused_smem + F_Q_AT + item * FQROW : fused_smem + F_NEW_AT;
            *(uint2*)(row + 8 * quad) = low;
            *(uint2*)(row + 2 * HALF + 8 * quad) = high;
            if (item == rows) {
                *(uint2*)(k_cache + new_at + 4 * quad) = low;
                *(uint2*)(k_cache + new_at + HALF + 4 * quad) = high;
            }
        }
        if (owns_newest) {
            // the new value row (not rotated); or, for a layer that reads a cache which another layer of this
            // step has written, that row and its key as they now stand in the cache
            for (int i = threadIdx.x; i < (write_kv ? 1 : 2) * (FHD / 4); i += FTHREADS) {
                const int which = write_kv ? 1 : i / (FHD / 4), quad = i % (FHD / 4);
                uint2 packed;
                if (write_kv) {
                    const float4 v = *(const float4*)(token + q_dim + kv_dim + (size_t)kv_head * FHD + 4 * quad);
                    packed = make_uint2(f_pack(v.x, v.y), f_pack(v.z, v.w));
                    *(uint2*)(v_cache + new_at + 4 * quad) = packed;
                } else {
                    packed = *(const uint2*)((which ? v_cache : k_cache) + new_at + 4 * quad);
                }
                *(uint2*)(fused_smem + F_NEW_AT + which * FQROW + 8 * quad) = packed;
            }
        }
    }
    __syncthreads();

    // query fragments: rows g and g+8 are heads head0+g, head0+g+8
    uint32_t qa[FKSTEPS][4];
#pragma unroll
    for (int s = 0; s < FKSTEPS; ++s)
        f_ldmatrix(qa[s], smem + F_Q_AT + ((lane & 7) + ((lane >> 3) & 1) * 8) * FQROW + (16 * s + (lane >> 4) * 8) * 2);

    float o[FOTILES][4];
#pragma unroll
    for (int j = 0; j < FOTILES; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};

    for (int c = 0; c < n_chunks; ++c) {
        // chunk c has landed (this thread's part) once all but the stages - 1 groups committed after it are complete
        if (stages == 2) f_wait_copies<1>();
        else if (stages == 3) f_wait_copies<2>();
        else f_wait_copies<3>();
        __syncthreads();                              // ... and everybody's
        const int group0 = my_first + c * FWARPS;
        const uint32_t stage = smem + F_STAGES_AT + (c % stages) * FSTAGE_BYTES;
        if (owns_newest && newest_group >= group0 && newest_group < group0 + FWARPS) {
            // the newest position's row, which the copy fetched as the cache had it before this step
            const int row = pos - (group0 << 4);
            unsigned char* base = fused_smem + F_STAGES_AT + (c % stages) * FSTAGE_BYTES;
            for (int i = threadIdx.x; i < 2 * FPIECES; i += FTHREADS) {
                const int which = i / FPIECES, piece = i - which * FPIECES;
                *(uint4*)(base + which * FCHUNK * FROW + f_staged(row, piece)) =
                    *(const uint4*)(fused_smem + F_NEW_AT + which * FQROW + piece * 16);
            }
            __syncthreads();
        }
        const int group = group0 + warp;
        if (group < my_end) {
            const int j0 = group << 4;
            const uint32_t k_rows = stage + warp * 16 * FROW, v_rows = k_rows + FCHUNK * FROW;
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
            for (int step = 0; step < FKSTEPS; ++step) {
                uint32_t kb[4];                       // keys 0-7: dims 0-7, 8-15 of the step; keys 8-15 likewise
                f_ldmatrix(kb, k_rows + f_staged((lane & 7) + (lane >> 4) * 8, 2 * step + ((lane >> 3) & 1)));
                f_mma(s[0], qa[step][0], qa[step][1], qa[step][2], qa[step][3], kb[0], kb[1]);
                f_mma(s[1], qa[step][0], qa[step][1], qa[step][2], qa[step][3], kb[2], kb[3]);
            }
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int t = 0; t < 2; ++t) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = j0 + 8 * t + 2 * tig + (e & 1);
                    const float v = (key < ctx && key >= lo) ? s[t][e] * scale_log2 : -INFINITY;
                    s[t][e] = v;
                    tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                }
            }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float m = tile_max[r];
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                const float new_max = fmaxf(row_max[r], m);
                corr[r] = new_max == -INFINITY ? 1.0f : f_exp2(row_max[r] - new_max);
                row_max[r] = new_max;
            }
            float p[2][4];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float m = row_max[e >> 1];
                    p[t][e] = m == -INFINITY ? 0.0f : f_exp2(s[t][e] - m);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r)
                row_sum[r] = row_sum[r] * corr[r] + p[0][2 * r] + p[0][2 * r + 1] + p[1][2 * r] + p[1][2 * r + 1];
#pragma unroll
            for (int j = 0; j < FOTILES; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            const uint32_t a0 = f_pack(p[0][0], p[0][1]), a1 = f_pack(p[0][2], p[0][3]);
            const uint32_t a2 = f_pack(p[1][0], p[1][1]), a3 = f_pack(p[1][2], p[1][3]);
#pragma unroll
            for (int j = 0; j < FOTILES; j += 2) {
                uint32_t vb[4];                       // dims 8j..: keys 0-7, 8-15; dims 8j+8..: keys 0-7, 8-15
                f_ldmatrix_trans(vb, v_rows + f_staged((lane & 7) + ((lane >> 3) & 1) * 8, j + (lane >> 4)));
                f_mma(o[j], a0, a1, a2, a3, vb[0], vb[1]);
                f_mma(o[j + 1], a0, a1, a2, a3, vb[2], vb[3]);
            }
        }
        __syncthreads();                              // the stage is free
        issue_chunk(c + stages);
    }
    f_wait_copies<0>();
    __syncthreads();

    // the warps' partial rows (outputs, max, sum), in what were the stages
    float* partial = (float*)(fused_smem + F_STAGES_AT);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    float* mine = partial + (size_t)warp * 16 * FPITCH;
#pragma unroll
    for (int j = 0; j < FOTILES; ++j) {
        mine[g * FPITCH + 8 * j + 2 * tig] = o[j][0];
        mine[g * FPITCH + 8 * j + 2 * tig + 1] = o[j][1];
        mine[(g + 8) * FPITCH + 8 * j + 2 * tig] = o[j][2];
        mine[(g + 8) * FPITCH + 8 * j + 2 * tig + 1] = o[j][3];
    }
    if (tig == 0) {
        mine[g * FPITCH + FHD] = row_max[0];
        mine[g * FPITCH + FHD + 1] = row_sum[0];
        mine[(g + 8) * FPITCH + FHD] = row_max[1];
        mine[(g + 8) * FPITCH + FHD + 1] = row_sum[1];
    }
    __syncthreads();
    f_cluster_wait();                                 // every block of the cluster runs: its shared memory may be written

    // Merge the warps, and push each row to the block that owns it: row r belongs to block r % blocks and
    // lands in that block's inbox at [(r / blocks) * blocks + this block's rank].
    const int rank = (int)f_cluster_rank(), blocks = (int)f_cluster_size();
    const uint32_t inbox_local = smem + F_INBOX_AT;
    for (int idx = threadIdx.x; idx < rows * FPITCH; idx += FTHREADS) {
        const int r = idx / FPITCH, d = idx - r * FPITCH;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < FWARPS; ++w) m = fmaxf(m, partial[((size_t)w * 16 + r) * FPITCH + FHD]);
        float value = m;
        if (d != FHD) {
            value = 0.0f;
            if (m != -INFINITY) {
#pragma unroll
                for (int w = 0; w < FWARPS; ++w) {
                    const float* tile = partial + ((size_t)w * 16 + r) * FPITCH;
                    value += f_exp2(tile[FHD] - m) * tile[d];      // column FHD+1 (the sums) is weighted the same way
                }
            }
        }
        const int slot = (r / blocks) * blocks + rank;
        f_remote_store(f_remote(inbox_local + (slot * FPITCH + d) * 4, (uint32_t)(r % blocks)), value);
    }
    f_cluster_arrive();
    f_cluster_wait();                                 // the pushes are visible; nobody reads another block from here on

    for (int idx = threadIdx.x; idx < ((rows - rank + blocks - 1) / blocks) * FHD; idx += FTHREADS) {
        const int mine_index = idx / FHD, d = idx - mine_index * FHD;
        const int r = mine_index * blocks + rank;
        const float* slots = inbox + (size_t)mine_index * blocks * FPITCH;
        float m = -INFINITY;
        for (int b = 0; b < blocks; ++b) m = fmaxf(m, slots[b * FPITCH + FHD]);
        float total = 0.0f, sum = 0.0f;
        for (int b = 0; b < blocks; ++b) {
            const float mb = slots[b * FPITCH + FHD];
            if (mb == -INFINITY) continue;
            const float weight = f_exp2(mb - m);
            total += weight * slots[b * FPITCH + d];
            sum += weight * slots[b * FPITCH + FHD + 1];
        }
        out[((size_t)seq * num_heads + head0 + r) * FHD + d] = __float2bfloat16_rn(total / sum);
    }
}

}  // namespace skv

using namespace skv;

// qkv: float [n_seqs, (heads + 2 kv_heads) * head_dim] (the q|k|v projection of each sequence's new
// token); cos_sin: float [positions, head_dim/2, 2] or null; ctx_after[s]: keys cached for sequence s
// once this token's key is in (so the token's position is ctx_after[s] - 1).  splits is 1..8.
SKV_EXPORT int skv_attention_decode_fused(const float* qkv, const float* cos_sin, void* k_cache, void* v_cache,
                                          const int* block_table, int table_width, const int* ctx_after,
                                          void* out, int n_seqs, int num_heads, int num_kv_heads, int head_dim,
                                          int block_size, float scale, int window, int splits, int write_kv,
                                          cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (head_dim != FHD) return fail("skv_attention_decode_fused", "this library was built for another head size");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention_decode_fused", "heads must be a positive multiple of kv heads");
    if (block_size <= 0 || block_size % 16 != 0)
        return fail("skv_attention_decode_fused", "block_size must be a positive multiple of 16");
    if (splits < 1 || splits > 8) return fail("skv_attention_decode_fused", "splits must be 1..8 (one cluster)");
    if (((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)qkv) & 15)
        return fail("skv_attention_decode_fused", "operands must be 16-byte aligned");
    const int group_size = num_heads / num_kv_heads;
    const int m_tiles = (group_size + 15) / 16;
    int block_shift = -1;                             // log2 of block_size where it is a power of two
    for (int bit = 4; bit < 31; ++bit)
        if (block_size == (1 << bit)) block_shift = bit;
    static int sm_count = 0;
    if (sm_count == 0) {
        int device = 0, count = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
            return fail("skv_attention_decode_fused", "cannot read the number of SMs");
        const cudaError_t status = cudaFuncSetAttribute(decode_attention_fused_kernel,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM_LIMIT);
        if (status != cudaSuccess) return fail("skv_attention_decode_fused", cudaGetErrorString(status));
        sm_count = count;
    }
    // Two stages of 128 keys let two blocks share an SM.  A block that has an SM to itself, and whose piece of
    // the longest context is at most four stages, fetches the whole piece ahead instead (measured: batch 8 at
    // 2,048 keys gains 3 % that way, while deeper staging of longer pieces loses 10 %).
    const long long blocks = (long long)n_seqs * num_kv_heads * m_tiles * splits;
    const long long piece_chunks = ((long long)table_width * block_size / splits + FCHUNK - 1) / FCHUNK;
    const int room = (F_SMEM_LIMIT - F_STAGES_AT) / FSTAGE_BYTES;
    // (a third stage for longer pieces, which two blocks of head size 64 could still share an SM with, measured
    // 7-12 % slower in the step at 8,100 and 16,200 keys)
    int stages = 2;
    if (blocks <= sm_count && piece_chunks <= FMAX_STAGES && piece_chunks <= room) stages = (int)(piece_chunks < 2 ? 2 : piece_chunks);
    const size_t smem = (size_t)F_STAGES_AT + (size_t)stages * FSTAGE_BYTES;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(n_seqs, num_kv_heads * m_tiles, splits);
    config.blockDim = dim3(FTHREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 1;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = splits;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    const cudaError_t status = cudaLaunchKernelEx(
        &config, decode_attention_fused_kernel, qkv, (const float2*)cos_sin, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, block_table, table_width, ctx_after, (__nv_bfloat16*)out, num_heads, num_kv_heads,
        block_size, scale, window, splits, m_tiles, write_kv, block_shift, stages);
    if (status != cudaSuccess) return fail("skv_attention_decode_fused", cudaGetErrorString(status));
    return 0;
}

SKV_EXPORT int skv_has_attention_decode_fused() { return 1; }

#else

SKV_EXPORT int skv_attention_decode_fused(const float*, const float*, void*, void*, const int*, int, const int*, void*,
                                          int, int, int, int, int, float, int, int, int, cudaStream_t) {
    return skv::fail("skv_attention_decode_fused",
                     "this kernel exists in the bfloat16 build for head sizes up to 192 only");
}

SKV_EXPORT int skv_has_attention_decode_fused() { return 0; }

#endif
