// Causal attention for prompt portions on the fifth-generation tensor cores, reading keys
// and values from the paged cache.
//
// One CTA takes 128 consecutive tokens of one request (a "tile" of queries) and one head.
// For every block of 128 keys up to the tile's last position:
//   producer warp   TMA-loads the block's keys and values page by page (the block table
//                   names the pages) into shared memory, 128-byte swizzle;
//   MMA warp        S = Q K^T with tcgen05.mma into tensor memory, later O_blk = P V;
//   softmax warps   two threads per query row read their halves of its row of S, apply
//                   scale, causal (and window) mask and the online softmax in 32-bit, writes
//                   P as bfloat16 into shared memory for the second product, and folds
//                   O_blk into its running output row with the usual rescaling.
// The reference's prefill attention is one thread per (query, head) walking all keys serially
// with the same online softmax (engine/src/attention.cu:71-124); its math is kept, the
// products move to the tensor cores.
//
// S has two buffers in tensor memory: S of block j+1 is computed while the softmax warps work
// on block j.  The block's output O_blk = P V is written over the S buffer that was just
// read, and folded into the running output one block later (behind the next block's row
// maxima), so that neither product is waited for.  Keys and values have barriers of their
// own: the keys of block j+2 are loaded as soon as S of block j is done.
//
// A tile with many key blocks may be given to several CTAs ("parts"), each taking a share of
// the blocks: the work list names part and number of parts.  A part leaves its un-normalised
// output, maximum and sum in scratch memory; the part that arrives last adds them in the order
// of the parts and writes the tile.  The longest CTA then has a few blocks, not all of them.
//
// The CTAs are persistent: two per SM (256 TMEM columns and ~115 KB of shared memory each;
// while one waits for its softmax the other's products run), each taking the next record of
// the work list from a counter until the list is done.  The list is sorted by falling number
// of key blocks, so that the long tiles start first and the short ones fill the gaps; tensor
// memory is allocated once per CTA.  Every mbarrier wait is bounded (tcgen05.cuh).
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

MLLM_DEFINE_ERROR_API(mllm_attention)

namespace {

constexpr int TILE = 128;          // queries per CTA = keys per block = TMEM lanes
constexpr int KV_STAGES = 2;
constexpr int THREADS = 320;       // warps 0-7 softmax, 8 producer, 9 MMA
constexpr int TMEM_COLS = 256;     // two S buffers of 128 columns; O_blk of block j overwrites S of block j

// 2^x with the hardware's approximation (about 2 ulp): its results are rounded to bfloat16.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The largest of three in one instruction (sm_100 has it): a row's maximum in half the instructions.
__device__ __forceinline__ float max_of_three(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

struct AttentionParams {
    bf16* out;                     // [T, ld_out]
    long ld_out;
    const int* tiles;              // per CTA: item, first row, rows, position of the first row, part,
                                   // parts, number of the tile among the split ones, unused
    float* partial;                // [split tiles, heads, max_parts, 128, D + 4]: a part's output, maximum, sum, padding
    int* counters;                 // [split tiles, heads], zero between launches
    int max_parts;
    int n_tiles;                   // records of the work list
    int* work;                     // [2] zero between launches: next (record, head) to take; CTAs that are done
    const int* block_table;        // [items, max_blocks]
    int max_blocks;
    int n_heads, n_kv_heads;
    int page_size, n_pages;
    float scale_log2;              // score scale * log2(e)
    int window;                    // 0: all keys
    int* status;
};

template <int D>
__global__ void __launch_bounds__(THREADS, D <= 64 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const AttentionParams p) {
    constexpr int DB = D / 64;                     // 64-column blocks of the head size
    constexpr int TILE_BYTES = TILE * 64 * 2;      // one [128 x 64] bf16 block, 16 KB
    // Swizzled tiles start on 1024-byte boundaries.  There is no static shared memory in this
    // kernel, so the dynamic part starts the CTA's window; should it ever not be aligned, the
    // CTA reports that and does nothing (two CTAs per SM leave no room for slack).
    extern __shared__ __align__(1024) unsigned char smem[];
    dependents_may_start();
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(p.status, 14);
        return;
    }
    unsigned char* q_tile = smem;                                   // DB blocks
    unsigned char* k_stage = q_tile + DB * TILE_BYTES;              // KV_STAGES x DB blocks
    unsigned char* v_stage = k_stage + KV_STAGES * DB * TILE_BYTES; // KV_STAGES x DB blocks
    unsigned char* p_tile = v_stage + KV_STAGES * DB * TILE_BYTES;  // 2 blocks: keys 0..63, 64..127
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_tile + 2 * TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;                   // [KV_STAGES]
    uint64_t* k_empty = k_full + KV_STAGES;        // [KV_STAGES]
    uint64_t* v_full = k_empty + KV_STAGES;        // [KV_STAGES]
    uint64_t* v_empty = v_full + KV_STAGES;        // [KV_STAGES]
    uint64_t* s_ready = v_empty + KV_STAGES;       // [2]: S of an even / odd block is in tensor memory
    uint64_t* o_ready = s_ready + 2;               // [2]: O_blk of an even / odd block is in tensor memory
    uint64_t* o_folded = o_ready + 2;              // [2]: every softmax warp has read that O_blk
    uint64_t* p_ready = o_folded + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_ready + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // the halves' maxima of each row [2][128]; bfloat16 is enough (both halves read the same
    // rounded values, and the maximum only anchors the exponentials) and all that fits
    bf16* row_max = reinterpret_cast<bf16*>(tmem_slot + 2);

    int* next_work = reinterpret_cast<int*>(row_max + 2 * 128);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pages_per_block = TILE / p.page_size;
    if (threadIdx.x == 0) *failed = 0;
    if (warp == 9) tmem_alloc(tmem_slot, TMEM_COLS);
    tcgen05_before_sync();
    __syncthreads();
    tcgen05_after_sync();
    const uint32_t tmem_base = *tmem_slot;         // buffer b: columns 128 b ..
    const int total_work = p.n_tiles * p.n_heads;
    wait_for_earlier_kernels();                    // nothing above reads or writes the step's memory

  for (int round = 0;; round++) {
    // ---- the next (record, head); fresh barriers for it ----
    if (threadIdx.x == 0) {
        *next_work = atomicAdd(p.work, 1);
        if (round > 0)
            for (int b = 0; b < 4 * KV_STAGES + 8; b++) mbar_inval(&bars[b]);
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&s_ready[b], 1);
            mbar_init(&o_ready[b], 1);
            mbar_init(&o_folded[b], 8);            // one arrival per softmax warp
        }
        mbar_init(p_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int work = *next_work;
    if (work >= total_work || *failed) break;
    const int* tile = p.tiles + 8 * (work / p.n_heads);
    const int item = tile[0], row0 = tile[1], n_rows = tile[2], pos0 = tile[3];
    const int part = tile[4], n_parts = tile[5], split_id = tile[6];
    const int head = work % p.n_heads;
    const int kv_head = head / (p.n_heads / p.n_kv_heads);
    const int last_pos = pos0 + n_rows - 1;
    const int first_key = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    // the key blocks of the tile, and this part's share of them (none, if a window left fewer
    // blocks than parts)
    const int tile_lo = first_key / TILE, tile_blocks = last_pos / TILE - tile_lo + 1;
    const int per_part = (tile_blocks + n_parts - 1) / n_parts;
    const int block_lo = tile_lo + part * per_part;
    const int n_blocks = max(0, min(per_part, tile_blocks - part * per_part));

    if (warp == 8) {
        // ---- producer ----
        if (lane == 0) {
            mbar_expect_tx(q_full, DB * TILE_BYTES);
            for (int db = 0; db < DB; db++)
                tma_load_2d(q_tile + db * TILE_BYTES, &map_q, q_full, head * D + db * 64, row0);
            const int* bt = p.block_table + (long)item * p.max_blocks;
            int issued_k = 0, issued_v = 0;
            for (int j = 0; j < n_blocks; j++) {
                const int s = j % KV_STAGES;
                const uint32_t parity = ((j / KV_STAGES) & 1) ^ 1;
                const int first_page = (block_lo + j) * pages_per_block;
                auto load = [&](unsigned char* stage, const CUtensorMap* map, uint64_t* full) {
                    mbar_expect_tx(full, DB * TILE_BYTES);
                    for (int g = 0; g < pages_per_block; g++) {
                        const int index = first_page + g;
                        // A page past the request's last one is read outside the pool: zeros.
                        int page = (index < p.max_blocks && index * p.page_size <= last_pos) ? bt[index] : -1;
                        if (page < 0) page = p.n_pages;
                        const int offset = g * p.page_size * 128;           // rows of 128 bytes
                        for (int db = 0; db < DB; db++)
                            tma_load_4d(stage + (s * DB + db) * TILE_BYTES + offset, map, full, db * 64, kv_head, 0, page);
                    }
                };
                if (!mbar_wait_idle(&k_empty[s], parity) || *failed) break;
                load(k_stage, &map_k, &k_full[s]);
                issued_k = j + 1;
                if (!mbar_wait_idle(&v_empty[s], parity) || *failed) break;
                load(v_stage, &map_v, &v_full[s]);
                issued_v = j + 1;
            }
            if (issued_v < n_blocks && !*failed) {
                *failed = 1;
                atomicExch(p.status, 11);
            }
            if (*failed) {
                // copies that were issued still land in shared memory: none may be in flight at the end
                mbar_wait(q_full, 0);
                for (int j = max(0, issued_k - KV_STAGES); j < issued_k; j++)
                    mbar_wait(&k_full[j % KV_STAGES], (j / KV_STAGES) & 1);
                for (int j = max(0, issued_v - KV_STAGES); j < issued_v; j++)
                    mbar_wait(&v_full[j % KV_STAGES], (j / KV_STAGES) & 1);
            }
        }
    } else if (warp == 9) {
        // ---- MMA issue ----
        if (lane == 0) {
            const uint32_t idesc_s = make_instr_desc(TILE, TILE);
            const uint32_t idesc_o = make_instr_desc(TILE, D) | IDESC_B_MN_MAJOR;
            bool ok = mbar_wait(q_full, 0);
            auto issue_s = [&](int j) {
                const int s = j % KV_STAGES;
                tcgen05_after_sync();
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; kk++) {
                    const uint64_t a = make_smem_desc(smem_u32(q_tile + (kk / 4) * TILE_BYTES)) + 2 * (kk % 4);
                    const uint64_t b = make_smem_desc(smem_u32(k_stage + (s * DB + kk / 4) * TILE_BYTES)) + 2 * (kk % 4);
                    umma(tmem_base + 128 * (j & 1), a, b, idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_ready[j & 1]);
                umma_commit(&k_empty[s]);
            };
            if (ok && n_blocks > 0) ok = mbar_wait(&k_full[0], 0);
            if (ok && n_blocks > 0) issue_s(0);
            for (int j = 0; ok && j < n_blocks; j++) {
                const int s = j % KV_STAGES;
                if (j + 1 < n_blocks) {
                    // S of the next block, while the softmax warps work on this one; its buffer
                    // held O_blk of block j-1, which every softmax warp must have read
                    ok = mbar_wait(&k_full[(j + 1) % KV_STAGES], ((j + 1) / KV_STAGES) & 1) && !*failed;
                    if (ok && j >= 1) ok = mbar_wait_idle(&o_folded[(j - 1) & 1], ((j - 1) >> 1) & 1) && !*failed;
                    if (!ok) break;
                    issue_s(j + 1);
                }
                // P is in shared memory and S of this block has been read: O_blk goes over S
                ok = mbar_wait_idle(p_ready, j & 1) && mbar_wait(&v_full[s], (j / KV_STAGES) & 1) && !*failed;
                if (!ok) break;
                tcgen05_after_sync();
#pragma unroll
                for (int kk = 0; kk < TILE / UMMA_K; kk++) {
                    const uint64_t a = make_smem_desc(smem_u32(p_tile + (kk / 4) * TILE_BYTES)) + 2 * (kk % 4);
                    // 16 keys = two 8-row groups of the value tile; head dims beyond 64 lie one tile further
                    const uint64_t b = make_smem_desc_mn(smem_u32(v_stage + s * DB * TILE_BYTES + kk * 2048), TILE_BYTES);
                    umma(tmem_base + 128 * (j & 1), a, b, idesc_o, kk > 0 ? 1u : 0u);
                }
                umma_commit(&o_ready[j & 1]);
                umma_commit(&v_empty[s]);
            }
            // the commits that free the last stages have arrived before the barriers are set up again
            for (int j = max(0, n_blocks - KV_STAGES); ok && j < n_blocks; j++)
                ok = mbar_wait(&k_empty[j % KV_STAGES], (j / KV_STAGES) & 1) &&
                     mbar_wait(&v_empty[j % KV_STAGES], (j / KV_STAGES) & 1);
            if (!ok && !*failed) {
                *failed = 1;
                atomicExch(p.status, 12);
            }
        }
    } else {
        // ---- softmax and output: two threads per query row, each half of the columns ----
        // Warp w reads TMEM lanes 32 (w % 4) ..; warps 0-3 take keys 0..63 of a block and the
        // first half of the head dims, warps 4-7 keys 64..127 and the second half.
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;
        const int my_pos = pos0 + min(r, n_rows - 1);
        const int my_first = (p.window > 0 && my_pos - p.window + 1 > 0) ? my_pos - p.window + 1 : 0;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        constexpr int DH = D / 2;
        float o[DH];
#pragma unroll
        for (int d = 0; d < DH; d++) o[d] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        float corr_prev = 0.0f;                       // the rescaling that goes with the block not yet folded
        bool ok = true;
        // o = o * corr + O_blk of block j (tensor memory buffer j & 1); then the buffer is free
        auto fold = [&](int j, float corr) -> bool {
            bool done = true;
            if (lane == 0) done = mbar_wait(&o_ready[j & 1], (j >> 1) & 1) && !*failed;
            done = __shfl_sync(0xffffffffu, done, 0);
            if (!done) return false;
            tcgen05_after_sync();
#pragma unroll
            for (int c = 0; c < DH; c += 32) {
                float v[32];
                tmem_load_32(tmem_base + 128 * (j & 1) + lane_addr + half * DH + c, v);
#pragma unroll
                for (int i = 0; i < 32; i++) o[c + i] = o[c + i] * corr + v[i];
            }
            tcgen05_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_folded[j & 1]);
            return true;
        };
        for (int j = 0; j < n_blocks; j++) {
            const uint32_t tmem_s = tmem_base + 128 * (j & 1);
            if (lane == 0) ok = mbar_wait(&s_ready[j & 1], (j >> 1) & 1) && !*failed;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tcgen05_after_sync();
            const int key0 = (block_lo + j) * TILE + half * 64;
            // a block whose last key no query of the tile may see needs the mask; so does any window
            const bool needs_mask = (block_lo + j) * TILE + TILE - 1 > pos0 || p.window > 0;
            // pass 1: the maximum of this thread's half of the row, then of the whole row
            float half_max = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 64; c += 32) {
                float v[32];
                tmem_load_32(tmem_s + lane_addr + half * 64 + c, v);
                if (needs_mask) {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int key = key0 + c + i;
                        if (key <= my_pos && key >= my_first) half_max = fmaxf(half_max, v[i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) half_max = fmaxf(half_max, v[i]);
                }
            }
            row_max[half * 128 + r] = __float2bfloat16_rn(half_max);
            asm volatile("bar.sync 1, 256;" ::: "memory");     // the next write comes after the barrier below
            const float block_max = fmaxf(__bfloat162float(row_max[half * 128 + r]),
                                          __bfloat162float(row_max[(half ^ 1) * 128 + r]));
            const float m_new = fmaxf(m, block_max * p.scale_log2);
            const float corr = (m == -INFINITY) ? 0.0f : fast_exp2(m - m_new);
            const float base = (m_new == -INFINITY) ? 0.0f : m_new;
            // the block before: its product has had the first pass to finish, and the P tile
            // it read is written again below
            if (j > 0) {
                ok = fold(j - 1, corr_prev);
                if (!ok) break;
            }
            corr_prev = corr;
            // pass 2: probabilities, as bfloat16 into shared memory (swizzled like a TMA tile);
            // this thread's 64 keys are one 128-byte row of key block `half`
            float row_sum = 0.0f;
            unsigned char* block = p_tile + half * TILE_BYTES + r * 128;
#pragma unroll 1
            for (int c = 0; c < 64; c += 32) {
                float v[32];
                tmem_load_32(tmem_s + lane_addr + half * 64 + c, v);
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float e0 = fast_exp2(v[i] * p.scale_log2 - base), e1 = fast_exp2(v[i + 1] * p.scale_log2 - base);
                    if (needs_mask) {
                        const int key = key0 + c + i;
                        if (!(key <= my_pos && key >= my_first)) e0 = 0.0f;
                        if (!(key + 1 <= my_pos && key + 1 >= my_first)) e1 = 0.0f;
                    }
                    __nv_bfloat162 two = __floats2bfloat162_rn(e0, e1);
                    // the sum uses the rounded values the second product will see
                    row_sum += __low2float(two) + __high2float(two);
                    packed[i / 2] = *reinterpret_cast<uint32_t*>(&two);
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int chunk = (c / 8 + q) ^ (r & 7);
                    *reinterpret_cast<uint4*>(block + chunk * 16) =
                        make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
            l = l * corr + row_sum;
            m = m_new;
            // hand P to the tensor core: writes visible to the async proxy, all 128 rows done,
            // and S of this block read by everyone (its buffer takes O_blk next)
            fence_async_smem();
            tcgen05_before_sync();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (threadIdx.x == 0) mbar_arrive(p_ready);
        }
        if (ok && n_blocks > 0) ok = fold(n_blocks - 1, corr_prev);
        if (!ok) {
            if (lane == 0 && !*failed) {
                *failed = 1;
                atomicExch(p.status, 13);
            }
        } else {
            // the two halves of a row add their sums (through the P tile, free by now)
            float* sums = reinterpret_cast<float*>(p_tile);
            sums[half * 128 + r] = l;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            float total = l + sums[(half ^ 1) * 128 + r];
            bool writes = true;
            if (n_parts > 1) {
                // leave this part's state; the part that arrives last merges all of them
                constexpr int ROW = D + 4;              // rows stay 16-byte aligned for the float4 accesses
                float* mine = p.partial + (((long)split_id * p.n_heads + head) * p.max_parts + part) * (TILE * ROW) + r * ROW;
#pragma unroll
                for (int d = 0; d < DH; d += 4)
                    __stcg(reinterpret_cast<float4*>(mine + half * DH + d), make_float4(o[d], o[d + 1], o[d + 2], o[d + 3]));
                if (half == 0) {
                    __stcg(mine + D, m);
                    __stcg(mine + D + 1, total);
                }
                __threadfence();
                asm volatile("bar.sync 1, 256;" ::: "memory");
                int* ticket = reinterpret_cast<int*>(p_tile) + 512;          // behind the 256 sums
                if (threadIdx.x == 0) *ticket = atomicAdd(p.counters + split_id * p.n_heads + head, 1);
                asm volatile("bar.sync 1, 256;" ::: "memory");
                writes = *ticket == n_parts - 1;
                if (writes) {
                    __threadfence();
                    const float* all = p.partial + ((long)split_id * p.n_heads + head) * p.max_parts * (TILE * ROW) + r * ROW;
                    float top = -INFINITY;
                    for (int q = 0; q < n_parts; q++) top = fmaxf(top, __ldcg(all + (long)q * TILE * ROW + D));
                    total = 0.0f;
#pragma unroll
                    for (int d = 0; d < DH; d++) o[d] = 0.0f;
                    for (int q = 0; q < n_parts; q++) {
                        const float* theirs = all + (long)q * TILE * ROW;
                        const float mq = __ldcg(theirs + D);
                        const float weight = (mq == -INFINITY) ? 0.0f : fast_exp2(mq - top);
                        total += __ldcg(theirs + D + 1) * weight;
#pragma unroll
                        for (int d = 0; d < DH; d += 4) {
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(theirs + half * DH + d));
                            o[d] += v.x * weight; o[d + 1] += v.y * weight; o[d + 2] += v.z * weight; o[d + 3] += v.w * weight;
                        }
                    }
                    if (threadIdx.x == 0) p.counters[split_id * p.n_heads + head] = 0;     // ready for the next launch
                }
            }
            const float inv = 1.0f / total;
            if (writes && r < n_rows) {
                bf16* dst = p.out + (long)(row0 + r) * p.ld_out + (long)head * D + half * DH;
#pragma unroll
                for (int d = 0; d < DH; d += 8) {
                    uint32_t packed[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        __nv_bfloat162 two = __floats2bfloat162_rn(o[d + 2 * i] * inv, o[d + 2 * i + 1] * inv);
                        packed[i] = *reinterpret_cast<uint32_t*>(&two);
                    }
                    *reinterpret_cast<uint4*>(dst + d) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
            }
        }
    }

    // everyone is done with this record's barriers, tiles and tensor memory
    tcgen05_before_sync();
    __syncthreads();
    tcgen05_after_sync();
  }

    // the CTA that leaves last puts the counters back for the next launch
    if (threadIdx.x == 0) {
        const int left = atomicAdd(p.work + 1, 1);
        if (left == (int)gridDim.x - 1) {
            p.work[0] = 0;
            p.work[1] = 0;
        }
    }
    tcgen05_before_sync();
    __syncthreads();
    if (warp == 9) tmem_free(tmem_base, TMEM_COLS);
}

// ---- two tiles of queries per CTA -----------------------------------------------------------
//
// For steps with long prompt portions.  A unit of work is up to 256 consecutive tokens of one
// request (tile A: the first 128, tile B: the rest) and one head; both tiles run against one
// stream of key and value blocks, which is therefore loaded once for 256 queries.  Each tile
// has four softmax warps of its own with ONE thread per query row.  Per block of 128 keys the
// thread takes its whole row of S out of tensor memory in one load (after which S of the next
// block may be computed there), finds the row's maximum without asking another thread, and
// writes the probabilities as bfloat16 into shared memory for the second product.  The
// output stays in tensor memory: O += P V accumulates there over all blocks, and is taken
// out once, at the end; when a row's maximum grows, the row of O there is scaled down first.
// While one tile's threads compute exponentials the other tile's products run.  One CTA per
// SM (384 columns of tensor memory, 197 KB of shared memory).
//
//   producer warp   Q of both tiles, then K and V block by block (pages by TMA, as above)
//   MMA warps       one per tile; per block j: S of block j + 1 as soon as the tile's threads hold
//                   S of block j in registers; O += P V of block j as soon as its P is written
//   softmax warps   per tile and block: S into registers, row maximum, rescaling of O if the
//                   maximum grew, exponentials into P, row sum
//
// Tile A ends one block of keys before tile B where the causal mask leaves it nothing.  A unit
// with many key blocks may be given to several CTAs (parts), each with a share of the blocks,
// as above: with 256 queries a unit a step has few units, so that SMs are left for the parts of
// the long ones and the longest CTA of the step has half or a third of the blocks.
constexpr int WIDE_STAGES = 3;
constexpr int WIDE_TMEM_COLS = 512;                // (a power of two; 384 are used)
constexpr int WIDE_TILE_COLS = 192;                // per tile: S (128 columns), then O (64)
constexpr float RAISE_AFTER = 8.0f;                // see the softmax warps

constexpr int WIDE_THREADS = THREADS + 32;         // warps 0-7 softmax, 8 producer, 9 and 10 MMA issue

template <int D>
__global__ void __launch_bounds__(WIDE_THREADS, 1)
attention_two_tiles_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                           const __grid_constant__ CUtensorMap map_v, const AttentionParams p) {
    static_assert(D == 64, "two tiles per CTA: head size 64");
    constexpr int TILE_BYTES = TILE * 64 * 2;      // one [128 x 64] bf16 block, 16 KB
    extern __shared__ __align__(1024) unsigned char smem[];
    dependents_may_start();
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(p.status, 14);
        return;
    }
    unsigned char* q_tile = smem;                                   // [2] tiles
    unsigned char* k_stage = q_tile + 2 * TILE_BYTES;               // [WIDE_STAGES]
    unsigned char* v_stage = k_stage + WIDE_STAGES * TILE_BYTES;    // [WIDE_STAGES]
    unsigned char* p_tile = v_stage + WIDE_STAGES * TILE_BYTES;     // [2 tiles][2 blocks: keys 0..63, 64..127]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_tile + 4 * TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;                   // [WIDE_STAGES]
    uint64_t* k_empty = k_full + WIDE_STAGES;
    uint64_t* v_full = k_empty + WIDE_STAGES;
    uint64_t* v_empty = v_full + WIDE_STAGES;
    uint64_t* s_ready = v_empty + WIDE_STAGES;     // [tile]: S of the next block is in tensor memory
    uint64_t* s_taken = s_ready + 2;               // [tile]: every softmax warp of the tile holds that S in registers
    uint64_t* p_ready = s_taken + 2;               // [tile]: P of the block is in shared memory (and O is scaled)
    uint64_t* o_ready = p_ready + 2;               // [tile]: O += P V of the block has finished
    uint64_t* exp_done = o_ready + 2;              // [tile]: every softmax warp of the tile has taken the block's exponentials
    constexpr int N_BARS = 1 + 4 * WIDE_STAGES + 10;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* next_work = reinterpret_cast<int*>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pages_per_block = TILE / p.page_size;
    if (threadIdx.x == 0) *failed = 0;
    if (warp == 9) tmem_alloc(tmem_slot, WIDE_TMEM_COLS);
    tcgen05_before_sync();
    __syncthreads();
    tcgen05_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int total_work = p.n_tiles * p.n_heads;
    wait_for_earlier_kernels();                    // nothing above reads or writes the step's memory

  for (int round = 0;; round++) {
    if (threadIdx.x == 0) {
        *next_work = atomicAdd(p.work, 1);
        if (round > 0)
            for (int b = 0; b < N_BARS; b++) mbar_inval(&bars[b]);
        mbar_init(q_full, 1);
        for (int s = 0; s < WIDE_STAGES; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 2);             // both issuing threads are done with the stage
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 2);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(&s_ready[t], 1);
            mbar_init(&s_taken[t], 4);             // one arrival per softmax warp of the tile
            mbar_init(&p_ready[t], 1);
            mbar_init(&o_ready[t], 1);
            mbar_init(&exp_done[t], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int work = *next_work;
    if (work >= total_work || *failed) break;
    const int* unit = p.tiles + 8 * (work / p.n_heads);
    const int item = unit[0], row0 = unit[1], n_rows = unit[2], pos0 = unit[3];
    const int part = unit[4], n_parts = unit[5], split_id = unit[6];
    const int head = work % p.n_heads;
    const int kv_head = head / (p.n_heads / p.n_kv_heads);
    const int rows_a = min(n_rows, TILE), rows_b = max(0, n_rows - TILE);
    const int last_pos = pos0 + n_rows - 1;
    const int first_key = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int block_lo = first_key / TILE;
    // key blocks of the unit and of each tile (tile A's last position lies 128 before tile B's);
    // this part's share of them starts at block part_lo of the unit
    const int unit_blocks = last_pos / TILE - block_lo + 1;
    const int per_part = (unit_blocks + n_parts - 1) / n_parts, part_lo = part * per_part;
    const int n_blocks = max(0, min(per_part, unit_blocks - part_lo));
    const int blocks_a = max(0, min(n_blocks, (pos0 + rows_a - 1) / TILE - block_lo + 1 - part_lo));
    const int blocks_b = rows_b > 0 ? n_blocks : 0;
    const int first_block = block_lo + part_lo;

    if (warp == 8) {
        // ---- producer ----
        if (lane == 0) {
            mbar_expect_tx(q_full, (rows_b > 0 ? 2 : 1) * TILE_BYTES);
            tma_load_2d(q_tile, &map_q, q_full, head * D, row0);
            if (rows_b > 0) tma_load_2d(q_tile + TILE_BYTES, &map_q, q_full, head * D, row0 + TILE);
            const int* bt = p.block_table + (long)item * p.max_blocks;
            int issued_k = 0, issued_v = 0;
            for (int j = 0; j < n_blocks; j++) {
                const int s = j % WIDE_STAGES;
                const uint32_t parity = ((j / WIDE_STAGES) & 1) ^ 1;
                const int first_page = (first_block + j) * pages_per_block;
                auto load = [&](unsigned char* stage, const CUtensorMap* map, uint64_t* full) {
                    mbar_expect_tx(full, TILE_BYTES);
                    for (int g = 0; g < pages_per_block; g++) {
                        const int index = first_page + g;
                        // A page past the request's last one is read outside the pool: zeros.
                        int page = (index < p.max_blocks && index * p.page_size <= last_pos) ? bt[index] : -1;
                        if (page < 0) page = p.n_pages;
                        tma_load_4d(stage + s * TILE_BYTES + g * p.page_size * 128, map, full, 0, kv_head, 0, page);
                    }
                };
                if (!mbar_wait_idle(&k_empty[s], parity) || *failed) break;
                load(k_stage, &map_k, &k_full[s]);
                issued_k = j + 1;
                if (!mbar_wait_idle(&v_empty[s], parity) || *failed) break;
                load(v_stage, &map_v, &v_full[s]);
                issued_v = j + 1;
            }
            if (issued_v < n_blocks && !*failed) {
                *failed = 1;
                atomicExch(p.status, 15);
            }
            if (*failed) {
                // copies that were issued still land in shared memory: none may be in flight at the end
                mbar_wait(q_full, 0);
                for (int j = max(0, issued_k - WIDE_STAGES); j < issued_k; j++)
                    mbar_wait(&k_full[j % WIDE_STAGES], (j / WIDE_STAGES) & 1);
                for (int j = max(0, issued_v - WIDE_STAGES); j < issued_v; j++)
                    mbar_wait(&v_full[j % WIDE_STAGES], (j / WIDE_STAGES) & 1);
            }
        }
    } else if (warp >= 9) {
        // ---- MMA issue: warp 9 for tile A, warp 10 for tile B, each at its tile's pace ----
        // Both walk all of the unit's blocks: where a tile has no keys left (tile A's last block,
        // a unit without tile B) its thread only hands the stages back, in step with the other.
        const int t = warp - 9;
        if (lane == 0) {
            const int my_blocks = t == 0 ? blocks_a : blocks_b;
            const uint32_t idesc_s = make_instr_desc(TILE, TILE);
            const uint32_t idesc_o = make_instr_desc(TILE, D) | IDESC_B_MN_MAJOR;
            const uint32_t tmem_s = tmem_base + WIDE_TILE_COLS * t, tmem_o = tmem_s + TILE;
            bool ok = mbar_wait(q_full, 0);
            // S of block j (the tile's threads hold S of block j - 1 in registers by then); after
            // that this thread needs the keys' stage no more
            auto issue_s = [&](int j) {
                const int s = j % WIDE_STAGES;
                ok = mbar_wait(&k_full[s], (j / WIDE_STAGES) & 1) && !*failed;
                if (!ok) return;
                if (j >= my_blocks) {
                    mbar_arrive(&k_empty[s]);
                    return;
                }
                if (j > 0) ok = mbar_wait(&s_taken[t], (j - 1) & 1) && !*failed;
                if (!ok) return;
                tcgen05_after_sync();
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; kk++) {
                    const uint64_t a = make_smem_desc(smem_u32(q_tile + t * TILE_BYTES)) + 2 * kk;
                    const uint64_t b = make_smem_desc(smem_u32(k_stage + s * TILE_BYTES)) + 2 * kk;
                    umma(tmem_s, a, b, idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_ready[t]);
                umma_commit(&k_empty[s]);
            };
            if (ok && n_blocks > 0) issue_s(0);
            for (int j = 0; ok && j < n_blocks; j++) {
                const int s = j % WIDE_STAGES;
                // S of the next block, while the softmax warps compute this one's exponentials
                if (j + 1 < n_blocks) issue_s(j + 1);
                if (!ok) break;
                ok = mbar_wait(&v_full[s], (j / WIDE_STAGES) & 1) && !*failed;
                if (!ok) break;
                if (j >= my_blocks) {
                    mbar_arrive(&v_empty[s]);
                    continue;
                }
                // P is in shared memory, and the row of O that needed it has been scaled: O += P V
                ok = mbar_wait_idle(&p_ready[t], j & 1) && !*failed;
                if (!ok) break;
                tcgen05_after_sync();
#pragma unroll
                for (int kk = 0; kk < TILE / UMMA_K; kk++) {
                    const uint64_t a = make_smem_desc(smem_u32(p_tile + (2 * t + kk / 4) * TILE_BYTES)) + 2 * (kk % 4);
                    // 16 keys = two 8-row groups of the value tile
                    const uint64_t b = make_smem_desc_mn(smem_u32(v_stage + s * TILE_BYTES + kk * 2048), TILE_BYTES);
                    umma(tmem_o, a, b, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&o_ready[t]);
                umma_commit(&v_empty[s]);
            }
            // the arrivals that free the last stages have come in before the barriers are set up again
            for (int j = max(0, n_blocks - WIDE_STAGES); ok && j < n_blocks; j++)
                ok = mbar_wait(&k_empty[j % WIDE_STAGES], (j / WIDE_STAGES) & 1) &&
                     mbar_wait(&v_empty[j % WIDE_STAGES], (j / WIDE_STAGES) & 1);
            if (!ok && !*failed) {
                *failed = 1;
                atomicExch(p.status, 16);
            }
        }
    } else {
        // ---- softmax and output: warps 0-3 tile A, 4-7 tile B; thread r of a tile owns query row r ----
        const int t = warp >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int my_blocks = t == 0 ? blocks_a : blocks_b, my_rows = t == 0 ? rows_a : rows_b;
        const int tile_pos0 = pos0 + t * TILE;
        const int my_pos = tile_pos0 + min(r, max(my_rows, 1) - 1);
        const int my_first = (p.window > 0 && my_pos - p.window + 1 > 0) ? my_pos - p.window + 1 : 0;
        const uint32_t tmem_s = tmem_base + WIDE_TILE_COLS * t + ((uint32_t)(quarter * 32) << 16);
        const uint32_t tmem_o = tmem_s + TILE;
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        auto wait_for = [&](uint64_t* bar, uint32_t parity) -> bool {
            // (every lane looks for itself: the barrier's word is one broadcast read, and a vote
            // keeps the warp together should the lanes' limits run out apart)
            const bool done = mbar_wait(bar, parity) && !*failed;
            return __all_sync(0xffffffffu, done);
        };
        for (int j = 0; j < my_blocks; j++) {
            ok = wait_for(&s_ready[t], j & 1);
            if (!ok) break;
            tcgen05_after_sync();
            float v[TILE];
            tmem_load_128(tmem_s, v);
            // S of the next block may take the place of this one
            tcgen05_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_taken[t]);
            const int key0 = (first_block + j) * TILE;
            // a block whose last key no query of the tile may see needs the mask; so does any window
            const bool needs_mask = key0 + TILE - 1 > tile_pos0 || p.window > 0;
            if (needs_mask) {
#pragma unroll
                for (int i = 0; i < TILE; i++) {
                    const int key = key0 + i;
                    if (!(key <= my_pos && key >= my_first)) v[i] = -INFINITY;
                }
            }
            // (eight maxima side by side: one chain of 128 dependent instructions would be the thread's longest wait)
            float top[8];
#pragma unroll
            for (int i = 0; i < 8; i++) top[i] = v[i];
#pragma unroll
            for (int i = 8; i < TILE; i += 16)
#pragma unroll
                for (int c = 0; c < 8; c++) top[c] = max_of_three(top[c], v[i + 2 * c], v[i + 2 * c + 1]);
            const float block_max = fmaxf(max_of_three(top[0], top[1], top[2]), max_of_three(top[3], top[4], top[5]));
            const float block_max_all = max_of_three(block_max, top[6], top[7]);
            // The exponentials are taken against m, a maximum that may be stale: it is raised (and
            // the row's sum and its row of O scaled down) only when the true maximum has grown
            // past it by more than 8 in the exponent, so a probability stays below 2^8 and the
            // scaling, which costs a round trip to tensor memory, becomes rare.
            const float seen = block_max_all * p.scale_log2;
            const bool raise = seen > m + RAISE_AFTER || m == -INFINITY;
            const float m_new = raise ? seen : m;
            const float corr = (!raise || m == -INFINITY) ? (raise ? 0.0f : 1.0f) : fast_exp2(m - m_new);
            const float base = (m_new == -INFINITY) ? 0.0f : m_new;
            // probabilities as bfloat16, first into registers (a masked score is -inf: its exponential is 0)
            uint32_t packed[TILE / 2];
            float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};     // (four sums side by side, as above)
            {
                // The two tiles take their exponentials in turn (A0 B0 A1 B1 ...): together they
                // would share the SM's exponential units and then both leave them idle while they
                // do the rest of a block; in turn, one tile's rest falls under the other's
                // exponentials (20.4 -> 19.3 us for two prompts of 1,024 tokens).  A tile waits
                // only for turns that the other tile does take.
                const int other_blocks = t == 0 ? blocks_b : blocks_a;
                const int need = t == 0 ? j - 1 : j;       // the other tile's block whose exponentials come before these
                if (need >= 0 && need < other_blocks) {
                    ok = wait_for(&exp_done[t ^ 1], need & 1);
                    if (!ok) break;
                }
            }
#pragma unroll
            for (int i = 0; i < TILE; i += 2) {
                const float e0 = fast_exp2(v[i] * p.scale_log2 - base), e1 = fast_exp2(v[i + 1] * p.scale_log2 - base);
                sums[(i / 2) & 3] += e0 + e1;
                __nv_bfloat162 two = __floats2bfloat162_rn(e0, e1);
                packed[i / 2] = *reinterpret_cast<uint32_t*>(&two);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&exp_done[t]);
            if (j > 0) {
                // the product of the block before has finished (it had the exponentials' time for
                // it): P may be written again, and O may be scaled down where a row's maximum rose
                ok = wait_for(&o_ready[t], (j - 1) & 1);
                if (!ok) break;
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
                    tcgen05_after_sync();
#pragma unroll 1
                    for (int d0 = 0; d0 < D; d0 += 32) {      // (in pieces: the probabilities fill the registers)
                        float o[32];
                        tmem_load_32(tmem_o + d0, o);
#pragma unroll
                        for (int d = 0; d < 32; d++) o[d] *= corr;
                        tmem_store_32(tmem_o + d0, o);
                    }
                }
            }
            // P into shared memory (swizzled like a TMA tile): keys 0..63 are this row's 128
            // bytes of the tile's first block, 64..127 of its second
#pragma unroll
            for (int c = 0; c < TILE; c += 8) {
                unsigned char* block = p_tile + (2 * t + c / 64) * TILE_BYTES + r * 128;
                const int chunk = ((c % 64) / 8) ^ (r & 7);
                *reinterpret_cast<uint4*>(block + chunk * 16) =
                    make_uint4(packed[c / 2], packed[c / 2 + 1], packed[c / 2 + 2], packed[c / 2 + 3]);
            }
            l = l * corr + ((sums[0] + sums[1]) + (sums[2] + sums[3]));
            m = m_new;
            // hand P to the tensor core: writes visible to the async proxy, O scaled, all 128 rows done
            fence_async_smem();
            tcgen05_before_sync();
            if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
            else asm volatile("bar.sync 2, 128;" ::: "memory");
            if (r == 0) mbar_arrive(&p_ready[t]);
        }
        if (ok && my_blocks > 0) ok = wait_for(&o_ready[t], (my_blocks - 1) & 1);
        if (!ok && lane == 0 && !*failed) {
            *failed = 1;
            atomicExch(p.status, 17);
        }
        {
            float o[D];
            if (ok && my_blocks > 0) {
                tcgen05_after_sync();
                tmem_load_64(tmem_o, o);           // (by whole warps, rows past the tile's last included)
            } else {
#pragma unroll
                for (int d = 0; d < D; d++) o[d] = 0.0f;
            }
            bool writes = ok;
            if (n_parts > 1) {
                // leave this part's state (its output, the maximum it is scaled by and its sum); the
                // part that arrives last merges all of them in their order: nothing depends on timing
                // (laid out [part][tile][D + 4 values][128 rows]: the rows of a warp lie side by side)
                constexpr int ROW = D + 4;
                const long cell = (long)split_id * p.n_heads + head;
                float* mine = p.partial + ((cell * p.max_parts + part) * 2 + t) * (ROW * TILE) + r;
#pragma unroll
                for (int d = 0; d < D; d++) __stcg(mine + d * TILE, o[d]);
                __stcg(mine + D * TILE, m);
                __stcg(mine + (D + 1) * TILE, l);
                // (each tile of the unit on its own: a counter and a barrier of the tile's four warps)
                __threadfence();
                int* const ticket = next_work + 1 + t;
                int* const counter = p.counters + 2 * cell + t;
                auto tile_barrier = [&]() {
                    if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
                    else asm volatile("bar.sync 2, 128;" ::: "memory");
                };
                tile_barrier();
                if (r == 0) *ticket = atomicAdd(counter, 1);
                tile_barrier();
                writes = ok && *ticket == n_parts - 1 && !*failed;
                if (writes) {
                    __threadfence();
                    const float* all = p.partial + (cell * p.max_parts * 2 + t) * (ROW * TILE) + r;
                    const long step = (long)2 * ROW * TILE;
                    if (n_parts == 2) {
                        // Two parts, the usual case: this thread still holds its own part, so one
                        // round trip to L2 brings all of the other.  The sum is written so that it
                        // has the same bits whichever of the two parts arrived last.
                        const float* other = all + (part ^ 1) * step;
                        float x[D];
#pragma unroll
                        for (int d = 0; d < D; d++) x[d] = __ldcg(other + d * TILE);
                        const float m_other = __ldcg(other + D * TILE), l_other = __ldcg(other + (D + 1) * TILE);
                        const float m0 = part == 0 ? m : m_other, m1 = part == 0 ? m_other : m;
                        const float l0 = part == 0 ? l : l_other, l1 = part == 0 ? l_other : l;
                        const float top = fmaxf(m0, m1);
                        const float w0 = (m0 == -INFINITY) ? 0.0f : fast_exp2(m0 - top);
                        const float w1 = (m1 == -INFINITY) ? 0.0f : fast_exp2(m1 - top);
                        l = fmaf(l1, w1, l0 * w0);
#pragma unroll
                        for (int d = 0; d < D; d++) o[d] = part == 0 ? fmaf(x[d], w1, o[d] * w0) : fmaf(o[d], w1, x[d] * w0);
                    } else {
                    float top = -INFINITY;
                    for (int q = 0; q < n_parts; q++) top = fmaxf(top, __ldcg(all + q * step + D * TILE));
                    l = 0.0f;
#pragma unroll
                    for (int d = 0; d < D; d++) o[d] = 0.0f;
                    for (int q = 0; q < n_parts; q++) {
                        const float* theirs = all + q * step;
                        float x[D];                     // (all loads of a part first: they are on their way together)
#pragma unroll
                        for (int d = 0; d < D; d++) x[d] = __ldcg(theirs + d * TILE);
                        const float mq = __ldcg(theirs + D * TILE);
                        const float weight = (mq == -INFINITY) ? 0.0f : fast_exp2(mq - top);
                        l += __ldcg(theirs + (D + 1) * TILE) * weight;
#pragma unroll
                        for (int d = 0; d < D; d++) o[d] += x[d] * weight;
                    }
                    }
                }
                if (r == 0 && *ticket == n_parts - 1) *counter = 0;     // ready for the next launch
            }
            if (writes && r < my_rows) {
                const float inv = 1.0f / l;
                bf16* dst = p.out + (long)(row0 + t * TILE + r) * p.ld_out + (long)head * D;
#pragma unroll
                for (int d = 0; d < D; d += 8) {
                    uint32_t packed[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        __nv_bfloat162 two = __floats2bfloat162_rn(o[d + 2 * i] * inv, o[d + 2 * i + 1] * inv);
                        packed[i] = *reinterpret_cast<uint32_t*>(&two);
                    }
                    *reinterpret_cast<uint4*>(dst + d) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
            }
        }
    }

    // everyone is done with this unit's barriers, tiles and tensor memory
    tcgen05_before_sync();
    __syncthreads();
    tcgen05_after_sync();
  }

    // the CTA that leaves last puts the counters back for the next launch
    if (threadIdx.x == 0) {
        const int left = atomicAdd(p.work + 1, 1);
        if (left == (int)gridDim.x - 1) {
            p.work[0] = 0;
            p.work[1] = 0;
        }
    }
    tcgen05_before_sync();
    __syncthreads();
    if (warp == 9) tmem_free(tmem_base, WIDE_TMEM_COLS);
}

// ---- host side -------------------------------------------------------------------------

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled g_encode = nullptr;
std::mutex g_lock;

int encoder() {
    if (g_encode != nullptr) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result) != cudaSuccess ||
        fn == nullptr || result != cudaDriverEntryPointSuccess)
        return fail("attention: the driver does not offer cuTensorMapEncodeTiled");
    g_encode = reinterpret_cast<EncodeTiled>(fn);
    return 0;
}

int encode(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
           const cuuint32_t* box) {
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_error_text, MLLM_ERROR_BUFFER, "attention: cuTensorMapEncodeTiled failed with code %d", (int)r);
        return 3;
    }
    return 0;
}

struct Key {
    const void* base;
    long a, b, c, d;
    bool operator==(const Key& o) const { return base == o.base && a == o.a && b == o.b && c == o.c && d == o.d; }
};
struct KeyHash {
    size_t operator()(const Key& k) const {
        size_t h = reinterpret_cast<size_t>(k.base);
        for (long v : {k.a, k.b, k.c, k.d}) h = h * 1000003u ^ (size_t)v;
        return h;
    }
};
std::unordered_map<Key, CUtensorMap, KeyHash> g_maps;

// queries: a [rows, cols] view with row stride ld; boxes of 128 rows x 64 columns
int query_map(const void* base, long rows, long cols, long ld, CUtensorMap* out) {
    Key key{base, rows, cols, ld, -1};
    auto found = g_maps.find(key);
    if (found != g_maps.end()) { *out = found->second; return 0; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)TILE};
    int rc = encode(out, base, 2, dims, strides, box);
    if (rc == 0) g_maps.emplace(key, *out);
    return rc;
}

// pages: [n_pages, page_size, kv_heads, head_size]; boxes of one page x one head x 64 columns
int page_map(const void* base, long n_pages, long page_size, long kv_heads, long head_size, CUtensorMap* out) {
    Key key{base, n_pages, page_size, kv_heads, head_size};
    auto found = g_maps.find(key);
    if (found != g_maps.end()) { *out = found->second; return 0; }
    cuuint64_t dims[4] = {(cuuint64_t)head_size, (cuuint64_t)kv_heads, (cuuint64_t)page_size, (cuuint64_t)n_pages};
    cuuint64_t strides[3] = {(cuuint64_t)head_size * 2, (cuuint64_t)kv_heads * head_size * 2,
                             (cuuint64_t)page_size * kv_heads * head_size * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)page_size, 1};
    int rc = encode(out, base, 4, dims, strides, box);
    if (rc == 0) g_maps.emplace(key, *out);
    return rc;
}

template <int D>
int launch(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v, const AttentionParams& p, int n_tiles,
           cudaStream_t s) {
    constexpr int DB = D / 64;
    constexpr size_t smem = (size_t)(DB + 2 * KV_STAGES * DB + 2) * TILE * 64 * 2 + (4 * KV_STAGES + 8) * 8 + 16 + 2 * 128 * 2 + 16;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
            return fail("attention: cannot raise the shared memory limit");
        configured = true;
    }
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        sms = 148;
    const long total = (long)n_tiles * p.n_heads, resident = (long)sms * (D <= 64 ? 2 : 1);
    const cudaError_t launch_error = launch_kernel(g_dependent_launch != 0, attention_tcgen05_kernel<D>,
                                                   dim3((unsigned)std::min(total, resident)), dim3(THREADS), smem, s, q, k, v, p);
    return launched(launch_error, "attention_tcgen05_kernel");
}

template <int D>
int launch_two_tiles(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v, const AttentionParams& p, int n_units,
                     cudaStream_t s) {
    constexpr size_t smem = (size_t)(2 + 2 * WIDE_STAGES + 4) * TILE * 64 * 2 + (1 + 4 * WIDE_STAGES + 10) * 8 + 64;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_two_tiles_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
            return fail("attention: cannot raise the shared memory limit");
        configured = true;
    }
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        sms = 148;
    const long total = (long)n_units * p.n_heads;
    return launched(launch_kernel(g_dependent_launch != 0, attention_two_tiles_kernel<D>, dim3((unsigned)std::min(total, (long)sms)),
                                  dim3(WIDE_THREADS), smem, s, q, k, v, p),
                    "attention_two_tiles_kernel");
}

}  // namespace

// Whether the kernel takes a layout: head size 64 or 128, pages of 8, 16, 32, 64 or 128
// tokens, query rows that start on 16-byte boundaries.
extern "C" int mllm_attention_takes(int head_size, int page_size, long ld_q, const void* q) {
    const bool page_ok = page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
    return (head_size == 64 || head_size == 128) && page_ok && ld_q % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(q) & 15) == 0;
}

// tiles: device int32 [n_tiles, 8], one record per CTA = (entry of the step, first row among
// the step's tokens, rows (1..128), position of the first row, part, parts, number of the tile
// among the split ones, 0); rows of one tile belong to one request and are consecutive; a
// tile of several parts has one record per part.  partial / counters (may be null if no tile
// has parts): fp32 [split tiles, heads, max_parts, 128, head_size + 4] and zeroed int32
// [split tiles, heads] (the kernel leaves them zero).  work: two zeroed ints (left zero).
// The records should be sorted by falling number of key blocks.  status: zeroed device word,
// see the matrix-product kernel.
extern "C" int mllm_attention_prefill(void* out, long ld_out, const void* q, long q_rows, long q_cols, long ld_q,
                                      const void* k_pages, const void* v_pages, int n_pages, int page_size,
                                      const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                                      int n_heads, int n_kv_heads, int head_size, float scale, int window,
                                      int* status, float* partial, int* counters, int max_parts, int* work,
                                      void* stream) {
    if (n_tiles <= 0) return 0;
    if (work == nullptr) return fail("attention: the work counter is required");
    if (max_parts < 1 || (max_parts > 1 && (partial == nullptr || counters == nullptr)))
        return fail("attention: tiles in parts need scratch memory");
    if ((reinterpret_cast<uintptr_t>(partial) & 15) != 0) return fail("attention: the scratch must be 16-byte aligned");
    if (!mllm_attention_takes(head_size, page_size, ld_q, q))
        return fail("attention: head size must be 64 or 128, the page size a power of two in 8..128, q 16-byte aligned");
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535)
        return fail("attention: heads must be a multiple of key/value heads");
    if (ld_out % 8 != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
        return fail("attention: output rows must start on 16-byte boundaries");
    CUtensorMap map_q, map_k, map_v;
    {
        std::lock_guard<std::mutex> guard(g_lock);
        int rc = encoder();
        if (rc) return rc;
        if (g_maps.size() > 4096) g_maps.clear();
        rc = query_map(q, q_rows, q_cols, ld_q, &map_q);
        if (rc) return rc;
        rc = page_map(k_pages, n_pages, page_size, n_kv_heads, head_size, &map_k);
        if (rc) return rc;
        rc = page_map(v_pages, n_pages, page_size, n_kv_heads, head_size, &map_v);
        if (rc) return rc;
    }
    AttentionParams p{(bf16*)out, ld_out, tiles, partial, counters, max_parts, n_tiles, work, block_table, max_blocks, n_heads, n_kv_heads, page_size, n_pages,
                      scale * 1.4426950408889634f, window, status};
    cudaStream_t s = (cudaStream_t)stream;
    if (head_size == 64) return launch<64>(map_q, map_k, map_v, p, n_tiles, s);
    return launch<128>(map_q, map_k, map_v, p, n_tiles, s);
}

// The same for steps with long portions, two tiles of queries per CTA (head size 64 only).
// units: device int32 [n_units, 8], one record per CTA = (entry of the step, first row among
// the step's tokens, rows (1..256), position of the first row, part, parts, number of the unit
// among the split ones, 0); rows of one unit belong to one request and are consecutive; a unit
// of several parts (each a share of its key blocks) has one record per part.  partial /
// counters (may be null if no unit has parts): fp32 [split units, heads, max_parts, 256,
// head_size + 4] and zeroed int32 [split units, heads, 2] (left zero).  The records should be
// sorted by falling number of key blocks.  work: two zeroed ints (left zero).
extern "C" int mllm_attention_prefill_two_tiles(void* out, long ld_out, const void* q, long q_rows, long q_cols, long ld_q,
                                                const void* k_pages, const void* v_pages, int n_pages, int page_size,
                                                const int* block_table, int max_blocks, const int* units, int n_units,
                                                int n_heads, int n_kv_heads, int head_size, float scale, int window,
                                                int* status, float* partial, int* counters, int max_parts, int* work,
                                                void* stream) {
    if (n_units <= 0) return 0;
    if (work == nullptr) return fail("attention: the work counter is required");
    if (max_parts < 1 || (max_parts > 1 && (partial == nullptr || counters == nullptr)))
        return fail("attention: units in parts need scratch memory");
    if ((reinterpret_cast<uintptr_t>(partial) & 15) != 0) return fail("attention: the scratch must be 16-byte aligned");
    if (head_size != 64 || !mllm_attention_takes(head_size, page_size, ld_q, q))
        return fail("attention (two tiles): head size must be 64, the page size a power of two in 8..128, q 16-byte aligned");
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535)
        return fail("attention: heads must be a multiple of key/value heads");
    if (ld_out % 8 != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0)
        return fail("attention: output rows must start on 16-byte boundaries");
    CUtensorMap map_q, map_k, map_v;
    {
        std::lock_guard<std::mutex> guard(g_lock);
        int rc = encoder();
        if (rc) return rc;
        if (g_maps.size() > 4096) g_maps.clear();
        rc = query_map(q, q_rows, q_cols, ld_q, &map_q);
        if (rc) return rc;
        rc = page_map(k_pages, n_pages, page_size, n_kv_heads, head_size, &map_k);
        if (rc) return rc;
        rc = page_map(v_pages, n_pages, page_size, n_kv_heads, head_size, &map_v);
        if (rc) return rc;
    }
    AttentionParams p{(bf16*)out, ld_out, units, partial, counters, max_parts, n_units, work, block_table, max_blocks, n_heads,
                      n_kv_heads, page_size, n_pages, scale * 1.4426950408889634f, window, status};
    return launch_two_tiles<64>(map_q, map_k, map_v, p, n_units, (cudaStream_t)stream);
}
