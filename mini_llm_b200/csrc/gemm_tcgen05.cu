// Matrix products on the fifth-generation tensor cores: out = epilogue(x W^T + bias),
// bfloat16 operands, fp32 accumulation in tensor memory.
//
// Operand blocks of 64 along K come into a ring of shared-memory stages by TMA (128-byte
// swizzle) from a producer warp; one thread of the MMA warp issues tcgen05.mma on each filled
// stage (four K=16 instructions per block) and releases the stage with tcgen05.commit; eight
// epilogue warps read the accumulator from tensor memory with tcgen05.ld and fuse bias, gelu
// or the residual sum into the store.  The reference runs every prefill product as a naive
// one-thread-per-output kernel followed by separate bias, gelu and add launches
// (engine/src/matrixmult.cu:7-34, engine/src/linear.cu:9-18,
// engine/src/transformer_block.cu:153-202).
//
// Two kernels:
//   rows     (more than 64 tokens) tiles of 128 tokens x BN output features, walked by
//            persistent CTAs with two accumulators, so that a tile's epilogue runs under the
//            next tile's products; the fused query/key/value product scatters keys and values
//            straight into the cache pages.
//   swapped  (up to 64 tokens) the 128 tile rows are rows of W (output features), the BN
//            columns are tokens: a 128-row token tile would be mostly padding.  When such a
//            product has few tiles, each is shared along K by a cluster of CTAs.
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel writes a code to
// its status word, stops issuing work, waits (bounded again) for its own copies in flight,
// frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

MLLM_DEFINE_ERROR_API(mllm_gemm)

namespace {

constexpr int BM = 128;             // tile rows = TMEM lanes
constexpr int BK = 64;              // 64 bf16 = 128 bytes = one swizzle row
constexpr int THREADS = 320;        // warps 0-7 epilogue, 8 producer, 9 MMA (both kernels; a second issuing warp 10 where the rows kernel has one)
enum { STATUS_OK = 0, STATUS_TIMEOUT_PRODUCER = 1, STATUS_TIMEOUT_MMA = 2, STATUS_TIMEOUT_EPILOGUE = 3 };

struct GemmParams {
    void* out;                // bf16 or fp32 [rows of x, ldo]
    const float* bias;        // per output feature, or null
    int* status;              // device word, non-zero after a bounded wait ran out
    int M, N, K;              // rows of x, rows of W (output features), inner size
    long ldo;
    int epilogue;
    int out_f32;
    int splits;               // swapped orientation only: the CTAs of a cluster share a tile along K (blockIdx.z)
    // Optional scatter of a fused query/key/value product: output features below q_width go
    // to out [M, q_width], the next kv_width to the key pages, the rest to the value pages,
    // each token at the cache slot its position and block table name (k_pages null: off).
    bf16* k_pages;
    bf16* v_pages;
    const int* positions;
    const int* token_item;
    const int* block_table;
    int max_blocks, page_size, q_width, kv_width;
    // Optional (rows kernel): seven time stamps of CTA 0, in nanoseconds of %globaltimer: start,
    // set-up done, first operands landed, last product issued, first accumulator ready, first
    // epilogue done, end.  Null in the engine; measurements and a test pass a buffer.
    unsigned long long* timeline;
    int out_by_tma;           // rows kernel: blocks of `out` leave through shared memory and TMA (map_out is valid)
};

__device__ __forceinline__ float activate(float v, int epilogue) {
    if (epilogue == EPI_GELU_TANH) return gelu_tanh_fast(v);
    if (epilogue == EPI_GELU_ERF) return gelu_erf_f(v);
    return v;
}

// Thread block clusters: the CTAs that share a tile along K add their partial sums through
// each other's shared memory.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {       // by every thread of every CTA of the cluster
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float load_from_rank(const float* mine, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(mine)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

template <int EPI> __device__ __forceinline__ float activate_as(float v) {
    if (EPI == EPI_GELU_TANH) return gelu_tanh_fast(v);
    if (EPI == EPI_GELU_ERF) return gelu_erf_f(v);
    return v;
}

// One block of 32 rows x 32 columns, turned through shared memory (turn[r * 33 + c]), stored
// as bfloat16 with bias and activation; row r goes to base + row_offset(r).  When the block
// is whole and 4-byte aligned (paired), half a warp writes one row (two columns per lane, one
// 4-byte store), so an instruction covers two rows; otherwise one column per lane.
template <int EPI, typename RowOffset>
__device__ __forceinline__ void store_rows_bf16_as(const float* turn, bf16* base, RowOffset row_offset, bool paired,
                                                   bool col_ok, int lane, int rows_left, const float* bias) {
    if (paired) {
        const int half = lane >> 4, c = (lane & 15) * 2;
        const float b0 = bias != nullptr ? bias[c] : 0.0f, b1 = bias != nullptr ? bias[c + 1] : 0.0f;
#pragma unroll 4
        for (int r = half; r < 32; r += 2)
            if (r < rows_left) {
                const __nv_bfloat162 two = __floats2bfloat162_rn(activate_as<EPI>(turn[r * 33 + c] + b0),
                                                                 activate_as<EPI>(turn[r * 33 + c + 1] + b1));
                *reinterpret_cast<__nv_bfloat162*>(base + row_offset(r) + c) = two;
            }
    } else {
        const float b = (col_ok && bias != nullptr) ? bias[lane] : 0.0f;
#pragma unroll 4
        for (int r = 0; r < 32; r++)
            if (col_ok && r < rows_left)
                base[row_offset(r) + lane] = __float2bfloat16_rn(activate_as<EPI>(turn[r * 33 + lane] + b));
    }
}

// The activation is chosen outside the loops over the rows.
template <typename RowOffset>
__device__ __forceinline__ void store_rows_bf16(const float* turn, bf16* base, RowOffset row_offset, bool paired,
                                                bool col_ok, int lane, int rows_left, const float* bias, int epilogue) {
    if (epilogue == EPI_GELU_TANH) store_rows_bf16_as<EPI_GELU_TANH>(turn, base, row_offset, paired, col_ok, lane, rows_left, bias);
    else if (epilogue == EPI_GELU_ERF) store_rows_bf16_as<EPI_GELU_ERF>(turn, base, row_offset, paired, col_ok, lane, rows_left, bias);
    else store_rows_bf16_as<EPI_STORE>(turn, base, row_offset, paired, col_ok, lane, rows_left, bias);
}

// The end of a tile that the SPLITS CTAs of a cluster share along K.  Every CTA has left its
// partial sums in its shared memory ([token][128 features]); CTA `rank` finishes the tokens
// rank, rank + SPLITS, ...: thread (feature r, half) takes every other one of them.  All loads
// are asked for before any sum is formed: a load from another CTA's shared memory, and the old
// value of a residual sum from global memory, each take hundreds of cycles, and one after the
// other they were most of this kernel's time.  A CTA starts with its own part and goes round
// the cluster from there, so that the CTAs do not all read from the same one at once; the
// order of a sum depends on the token only, never on timing.
template <int BN, int SPLITS>
__device__ __forceinline__ void finish_split(const GemmParams& p, const float* part, const long* kv_off, float b, int r, int tile_b,
                                             int tokens, int rank, int half) {
    constexpr int MINE = (BN + 2 * SPLITS - 1) / (2 * SPLITS);      // this thread's tokens
    constexpr int PER = MINE < 64 / SPLITS ? MINE : 64 / SPLITS;      // of them at a time: 64 loads on their way
#pragma unroll 1
    for (int first = 0; first < MINE; first += PER) {
        const int c0 = rank + SPLITS * half + first * 2 * SPLITS;
        if (c0 >= tokens) break;
        float value[PER][SPLITS];
#pragma unroll
        for (int z = 0; z < SPLITS; z++)
#pragma unroll
            for (int i = 0; i < PER; i++) {
                const int c = c0 + i * 2 * SPLITS;
                value[i][z] = c < tokens ? load_from_rank(part + c * BM, (uint32_t)((rank + z) % SPLITS)) : 0.0f;
            }
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int c = c0 + i * 2 * SPLITS;
            if (c >= tokens) continue;
            float sum = 0.0f;
#pragma unroll
            for (int z = 0; z < SPLITS; z++) sum += value[i][z];
            const float x = sum + b;
            const int t = tile_b * BN + c;
            if (p.k_pages != nullptr && r >= p.q_width) {
                const long slot = kv_off[c];
                if (r < p.q_width + p.kv_width) p.k_pages[slot + r - p.q_width] = __float2bfloat16_rn(x);
                else p.v_pages[slot + r - p.q_width - p.kv_width] = __float2bfloat16_rn(x);
                continue;
            }
            const long at = (long)t * p.ldo + r;
            // (the residual sum as one addition at the memory: this thread is the only one that
            // adds to the element in this launch, and nothing waits for the old value)
            if (p.epilogue == EPI_ADD) atomicAdd(reinterpret_cast<float*>(p.out) + at, x);
            else if (p.out_f32) reinterpret_cast<float*>(p.out)[at] = x;
            else reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(activate(x, p.epilogue));
        }
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_swapped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    // map_a: W, whose rows (output features) fill the tile's 128 rows; map_b: x, BN tokens.
    extern __shared__ unsigned char smem_raw[];
    // The swizzled tiles must start on 1024-byte boundaries; the launch asks for 1024 spare bytes.
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    unsigned char* stage_a = smem;
    unsigned char* stage_b = smem + STAGES * A_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* accumulator_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accumulator_ready + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // element offset of each of the tile's tokens in the cache pages (scatter only)
    long* kv_off = reinterpret_cast<long*>(smem + STAGES * (A_BYTES + B_BYTES) + (2 * STAGES + 1) * 8 + 16);

    dependents_may_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_a = blockIdx.x;      // which block of 128 output features
    const int tile_b = blockIdx.y;      // which block of BN tokens
    // k blocks of this CTA: all of them, or its share when the tile is split along K
    const int all_k = (p.K + BK - 1) / BK;
    const int per_split = (all_k + p.splits - 1) / p.splits;
    const int kb_first = (int)blockIdx.z * per_split;
    const int num_k = max(0, min(all_k, kb_first + per_split) - kb_first);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accumulator_ready, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    wait_for_earlier_kernels();          // nothing above reads or writes the step's memory

    if (warp == 8) {
        // ---- producer ----
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < num_k; kb++) {
                const int s = kb % STAGES;
                if (!mbar_wait(&empty[s], ((kb / STAGES) & 1) ^ 1) || *failed) {
                    if (!*failed) {
                        *failed = STATUS_TIMEOUT_PRODUCER;
                        atomicExch(p.status, STATUS_TIMEOUT_PRODUCER);
                    }
                    break;
                }
                mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                tma_load_2d(stage_a + s * A_BYTES, &map_a, &full[s], (kb_first + kb) * BK, tile_a * BM);
                tma_load_2d(stage_b + s * B_BYTES, &map_b, &full[s], (kb_first + kb) * BK, tile_b * BN);
                issued = kb + 1;
            }
            if (*failed) {
                // Copies that were issued still land in shared memory: wait for them (bounded)
                // so that none is in flight when the CTA ends.
                for (int kb = max(0, issued - STAGES); kb < issued; kb++)
                    mbar_wait(&full[kb % STAGES], (kb / STAGES) & 1);
            }
        }
    } else if (warp == 9) {
        // ---- MMA issue ----
        if (lane == 0) {
            const uint32_t idesc = make_instr_desc(BM, BN);
            for (int kb = 0; kb < num_k; kb++) {
                const int s = kb % STAGES;
                if (!mbar_wait(&full[s], (kb / STAGES) & 1) || *failed) {
                    if (!*failed) {
                        *failed = STATUS_TIMEOUT_MMA;
                        atomicExch(p.status, STATUS_TIMEOUT_MMA);
                    }
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t desc_a = make_smem_desc(smem_u32(stage_a + s * A_BYTES));
                const uint64_t desc_b = make_smem_desc(smem_u32(stage_b + s * B_BYTES));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) {
                    // 16 elements along K = 32 bytes = 2 units of the descriptor's address field
                    umma(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);          // frees the stage once these MMAs have read it
            }
            umma_commit(accumulator_ready);      // arrives when every MMA above has finished
        }
    } else {
        // ---- epilogue: warps w and w + 4 own TMEM lanes 32w .. 32w+31 and split the columns ----
        const int quarter = warp & 3, col_half = warp >> 2;
        if (p.k_pages != nullptr) {
            const int t = tile_b * BN + threadIdx.x;
            if (t < p.M && threadIdx.x < BN) {
                const int pos = p.positions[t];
                const int page = p.block_table[(long)p.token_item[t] * p.max_blocks + pos / p.page_size];
                kv_off[threadIdx.x] = ((long)page * p.page_size + pos % p.page_size) * p.kv_width;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        bool ok = true;
        if (lane == 0) ok = mbar_wait(accumulator_ready, 0);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok || *failed) {
            if (lane == 0 && !*failed) {
                *failed = STATUS_TIMEOUT_EPILOGUE;
                atomicExch(p.status, STATUS_TIMEOUT_EPILOGUE);
            }
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int r = tile_a * BM + quarter * 32 + lane;       // row of map_a's operand
            const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
            // columns of this warp: one half of the tile (all of a tile narrower than 32)
            constexpr int SPAN = BN >= 32 ? BN / 2 : BN;
            const int c_first = BN >= 32 ? col_half * SPAN : 0;
            const bool has_columns = BN >= 32 || col_half == 0;
            {
                // r: an output feature; columns: tokens.  Consecutive lanes write consecutive
                // features of one token: coalesced.
                const bool row_ok = r < p.N;
                const float b = (row_ok && p.bias != nullptr) ? p.bias[r] : 0.0f;
                auto finish = [&](int t, float x) {
                    if (p.k_pages != nullptr && r >= p.q_width) {
                        const long slot = kv_off[t - tile_b * BN];
                        if (r < p.q_width + p.kv_width) p.k_pages[slot + r - p.q_width] = __float2bfloat16_rn(x);
                        else p.v_pages[slot + r - p.q_width - p.kv_width] = __float2bfloat16_rn(x);
                        return;
                    }
                    const long at = (long)t * p.ldo + r;
                    if (p.epilogue == EPI_ADD) reinterpret_cast<float*>(p.out)[at] += x;
                    else if (p.out_f32) reinterpret_cast<float*>(p.out)[at] = x;
                    else reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(activate(x, p.epilogue));
                };
                if (p.splits <= 1) {
#pragma unroll 1
                    for (int c0 = c_first; has_columns && c0 < c_first + SPAN; c0 += 16) {
                        float v[16];
                        __syncwarp();
                        tmem_load_16(lane_base + c0, v);
                        if (!row_ok) continue;
                        if (p.epilogue == EPI_ADD) {
                            // all old values first: sixteen loads in flight instead of one at a time
                            float* o = reinterpret_cast<float*>(p.out) + (long)(tile_b * BN + c0) * p.ldo + r;
                            const int left = p.M - (tile_b * BN + c0);
                            float old[16];
#pragma unroll
                            for (int i = 0; i < 16; i++) old[i] = i < left ? o[(long)i * p.ldo] : 0.0f;
#pragma unroll
                            for (int i = 0; i < 16; i++)
                                if (i < left) o[(long)i * p.ldo] = old[i] + v[i] + b;
                            continue;
                        }
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const int t = tile_b * BN + c0 + i;
                            if (t >= p.M) break;
                            finish(t, v[i] + b);
                        }
                    }
                } else {
                    // The tile is split along K over the CTAs of a cluster: every CTA leaves its
                    // partial sums in its own shared memory (the operand stages are free by
                    // now), [token][128 features]; they are added below, behind a cluster barrier.
                    float* part = reinterpret_cast<float*>(smem) + quarter * 32 + lane;
#pragma unroll 1
                    for (int c0 = c_first; has_columns && c0 < c_first + SPAN; c0 += 16) {
                        float v[16];
                        __syncwarp();
                        tmem_load_16(lane_base + c0, v);
#pragma unroll
                        for (int i = 0; i < 16; i++) part[(c0 + i) * BM] = num_k > 0 ? v[i] : 0.0f;
                    }
                }
            }
        }
    }

    if (p.splits > 1) {
        // Every thread of every CTA of the cluster comes by here, whatever happened above.
        __syncthreads();
        __syncwarp();
        cluster_sync();
        if (warp < 8 && !*failed) {
            // CTA `rank` finishes the tokens rank, rank + splits, ...: it adds the partial sums
            // of all CTAs in an order that the token fixes, so the result does not depend on
            // timing.  Thread t keeps feature t % 128 (the row it read from tensor memory).
            const int quarter = warp & 3;
            const int r = tile_a * BM + quarter * 32 + lane;
            const bool row_ok = r < p.N;
            const float b = (row_ok && p.bias != nullptr) ? p.bias[r] : 0.0f;
            const float* part = reinterpret_cast<const float*>(smem) + quarter * 32 + lane;
            const int tokens = min(BN, p.M - tile_b * BN), rank = (int)cluster_rank();
            if (row_ok) {
                switch (p.splits) {
                case 2: finish_split<BN, 2>(p, part, kv_off, b, r, tile_b, tokens, rank, warp >> 2); break;
                case 4: finish_split<BN, 4>(p, part, kv_off, b, r, tile_b, tokens, rank, warp >> 2); break;
                default: finish_split<BN, 8>(p, part, kv_off, b, r, tile_b, tokens, rank, warp >> 2); break;
                }
            }
        }
        __syncwarp();
        cluster_sync();        // nobody leaves while its shared memory may still be read
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 9) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

// ---- steps of many tokens: a persistent kernel ---------------------------------------------
//
// One CTA per SM walks tiles of 128 tokens x BN output features (tile t of CTA b is number
// b + t * gridDim.x; the row tile runs fastest, so CTAs that run side by side share a block
// of W in L2).  The producer warp keeps the ring of operand stages full across tile
// boundaries; the MMA thread accumulates tile t in one half of the allocated tensor memory
// while the eight epilogue warps drain tile t - 1 from the other half, so bias, activation,
// residual sum and the stores run under the next tile's products.  BN is 64, 96, 128, 192 or
// 256: wide tiles read less of x and W per output from L2 (what bounds these products),
// narrow ones spread a product with few output features over more SMs.
__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// A thread's 32 values of one row of the accumulator plus the 32 biases at shared address
// `bias32`, activated, as bfloat16 (EPI) or fp32 into this thread's row of a block in shared
// memory at address `dst` (rows of 64 or 128 bytes).
// The block is laid out as TMA's 64-byte (bfloat16) or 128-byte (fp32) swizzle reads it: the
// 16-byte piece j of row r lies at piece j ^ ((r / 2) % 4), respectively j ^ (r % 8), of its
// row, so that the lanes of a warp, each writing the same piece of its own row, hit different
// banks (all eight epilogue warps share one path into shared memory: a conflict costs them all).
template <int EPI>
__device__ __forceinline__ void stage_row_bf16(const float* v, uint32_t bias32, uint32_t block, int row) {
    const uint32_t dst = block + row * 64;
    const int twist = (row >> 1) & 3;
    float4 b[8];                                   // all loads first: they are in flight together
#pragma unroll
    for (int j = 0; j < 8; j++) b[j] = lds128(bias32 + j * 16);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float4 b0 = b[2 * j], b1 = b[2 * j + 1];
        const __nv_bfloat162 p0 = __floats2bfloat162_rn(activate_as<EPI>(v[8 * j] + b0.x), activate_as<EPI>(v[8 * j + 1] + b0.y));
        const __nv_bfloat162 p1 = __floats2bfloat162_rn(activate_as<EPI>(v[8 * j + 2] + b0.z), activate_as<EPI>(v[8 * j + 3] + b0.w));
        const __nv_bfloat162 p2 = __floats2bfloat162_rn(activate_as<EPI>(v[8 * j + 4] + b1.x), activate_as<EPI>(v[8 * j + 5] + b1.y));
        const __nv_bfloat162 p3 = __floats2bfloat162_rn(activate_as<EPI>(v[8 * j + 6] + b1.z), activate_as<EPI>(v[8 * j + 7] + b1.w));
        sts128(dst + ((j ^ twist) << 4), *reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1),
               *reinterpret_cast<const uint32_t*>(&p2), *reinterpret_cast<const uint32_t*>(&p3));
    }
}
__device__ __forceinline__ void stage_row_f32(const float* v, uint32_t bias32, uint32_t block, int row) {
    const uint32_t dst = block + row * 128;
    const int twist = row & 7;
    float4 b[8];
#pragma unroll
    for (int j = 0; j < 8; j++) b[j] = lds128(bias32 + j * 16);
#pragma unroll
    for (int j = 0; j < 8; j++)
        sts128(dst + ((j ^ twist) << 4), __float_as_uint(v[4 * j] + b[j].x), __float_as_uint(v[4 * j + 1] + b[j].y),
               __float_as_uint(v[4 * j + 2] + b[j].z), __float_as_uint(v[4 * j + 3] + b[j].w));
}

// (a block of 32 x 32 floats turned through shared memory, rows 33 floats apart, fits two of these)
constexpr int WARP_BLOCKS_BYTES = 2 * 4096;   // per epilogue warp: two blocks of 32 rows x 128 bytes for TMA, 1024-byte aligned
enum { STATUS_TIMEOUT_ROWS_PRODUCER = 5, STATUS_TIMEOUT_ROWS_MMA = 6, STATUS_TIMEOUT_ROWS_EPILOGUE = 7, STATUS_PAIR_TMEM_DIFFERS = 8 };


// Where an epilogue warp's blocks of 32 rows x 32 columns go, for finish_block().
struct BlockOut {
    const CUtensorMap* map_out;
    float* turn;               // the warp's two blocks of shared memory (8 KB, 1024-byte aligned)
    const float* bias_s;       // the tile's biases (zeros without a bias), in shared memory
    const long* kv_off;        // the tile's 128 cache offsets (scatter only)
    int quarter, lane;
    int boxes;                 // boxes this warp has sent: box b leaves from block b % 2
};

// One block of a tile's accumulator, v[i] = column c0 + i of this thread's row (row0 + lane),
// to where it belongs: bias, activation, conversion, and the way out.
__device__ __forceinline__ void finish_block(BlockOut& o, const GemmParams& p, const CUtensorMap& map_out, float* v, int c0,
                                             int n0, int row0) {
    float* turn = o.turn;
    const float* bias_s = o.bias_s;
    const long* kv_off = o.kv_off;
    const int quarter = o.quarter, lane = o.lane;
    int& boxes = o.boxes;
        const float* bs = bias_s + c0;
        const bool whole = n0 + 32 <= p.N;
        // Where the block of 32 x 32 goes.  A block of `out` leaves through shared memory
        // and one TMA box (stored, or added to what is there: the residual sum) when the
        // tensor is laid out for it.  A block of keys or values goes to scattered cache
        // slots: each thread stores its own row's 64 bytes from its registers.  Whatever
        // is laid out for neither is turned through shared memory, so that consecutive
        // lanes write consecutive columns.
        const bool wide = p.epilogue == EPI_ADD || p.out_f32;
        const int region = wide || p.k_pages == nullptr || n0 < p.q_width ? 0 : (n0 < p.q_width + p.kv_width ? 1 : 2);
        if (region == 0 && p.out_by_tma) {
            if (row0 >= p.M) return;
            if (lane == 0) bulk_wait_read_but_one();     // the box before the last one has left its block
            __syncwarp();
            unsigned char* mine = reinterpret_cast<unsigned char*>(turn) + (boxes & 1) * 4096;
            boxes++;
            const uint32_t bias32 = smem_u32(bs), block = smem_u32(mine);
            if (wide) stage_row_f32(v, bias32, block, lane);
            else if (p.epilogue == EPI_GELU_TANH) stage_row_bf16<EPI_GELU_TANH>(v, bias32, block, lane);
            else if (p.epilogue == EPI_GELU_ERF) stage_row_bf16<EPI_GELU_ERF>(v, bias32, block, lane);
            else stage_row_bf16<EPI_STORE>(v, bias32, block, lane);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                if (p.epilogue == EPI_ADD) tma_reduce_add_2d(&map_out, mine, n0, row0);
                else tma_store_2d(&map_out, mine, n0, row0);
                bulk_commit();
            }
            return;
        }
        if (region != 0 && whole && (p.kv_width & 7) == 0 &&
            (reinterpret_cast<uintptr_t>(region == 1 ? p.k_pages : p.v_pages) & 15) == 0) {
            // Keys or values: the block is staged as bfloat16 like a box, then four lanes
            // write one row's 64 bytes to its cache slot, eight rows per instruction.
            if (lane == 0) bulk_wait_read();
            __syncwarp();
            const uint32_t block = smem_u32(turn);
            stage_row_bf16<EPI_STORE>(v, smem_u32(bs), block, lane);
            __syncwarp();
            bf16* pages = region == 1 ? p.k_pages + (n0 - p.q_width) : p.v_pages + (n0 - p.q_width - p.kv_width);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = i * 8 + (lane >> 2), piece = lane & 3;
                const float4 x = lds128(block + row * 64 + ((piece ^ ((row >> 1) & 3)) << 4));
                if (row0 + row < p.M)
                    *reinterpret_cast<float4*>(pages + kv_off[quarter * 32 + row] + piece * 8) = x;
            }
            return;
        }
        if (lane == 0) bulk_wait_read();             // (a box may still be leaving the block)
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 32; i++) turn[lane * 33 + i] = v[i];
        __syncwarp();
        const int n = n0 + lane;
        const bool col_ok = n < p.N;
        const float b = col_ok ? bs[lane] : 0.0f;
        if (p.epilogue == EPI_ADD) {
            float* o = reinterpret_cast<float*>(p.out) + (long)row0 * p.ldo + n;
#pragma unroll 1
            for (int r0 = 0; r0 < 32; r0 += 8) {
                float old[8];
#pragma unroll
                for (int u = 0; u < 8; u++)
                    old[u] = (col_ok && row0 + r0 + u < p.M) ? o[(long)(r0 + u) * p.ldo] : 0.0f;
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (col_ok && row0 + r0 + u < p.M)
                        o[(long)(r0 + u) * p.ldo] = old[u] + turn[(r0 + u) * 33 + lane] + b;
            }
        } else if (p.out_f32) {
            float* o = reinterpret_cast<float*>(p.out) + (long)row0 * p.ldo + n;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr++)
                if (col_ok && row0 + rr < p.M) o[(long)rr * p.ldo] = turn[rr * 33 + lane] + b;
        } else {
            // bfloat16: rows of the output, or (scatter) slots of the cache pages
            bf16* const region_base = region == 0 ? reinterpret_cast<bf16*>(p.out) + (long)row0 * p.ldo + n0
                                      : (region == 1 ? p.k_pages + (n0 - p.q_width)
                                                     : p.v_pages + (n0 - p.q_width - p.kv_width));
            const bool paired = whole && (p.ldo & 1) == 0 && (p.kv_width & 1) == 0 &&
                                (reinterpret_cast<uintptr_t>(region_base) & 3) == 0;
            const long ldo = p.ldo;
            const long* slots = kv_off + quarter * 32;
            if (region == 0)
                store_rows_bf16(turn, region_base, [ldo](int rr) { return (long)rr * ldo; }, paired, col_ok, lane,
                                p.M - row0, p.bias != nullptr ? p.bias + n0 : nullptr, p.epilogue);
            else
                store_rows_bf16(turn, region_base, [slots](int rr) { return slots[rr]; }, paired, col_ok, lane,
                                p.M - row0, p.bias != nullptr ? p.bias + n0 : nullptr, p.epilogue);
        }
}

template <int BN, int STAGES, bool PAIR>
constexpr size_t rows_shared_bytes() {   // the same for one and for two issuing threads
    // stages, the epilogue warps' turning blocks, barriers, a few words, two sets of cache offsets, two of biases
    return (size_t)STAGES * (BM * BK * 2 + (PAIR ? BN / 2 : BN) * BK * 2) + 8 * WARP_BLOCKS_BYTES + (2 * STAGES + 6) * 8 + 16 +
           2 * BM * 8 + 2 * 256 * 4 + 1024;
}

// ISSUERS: the threads that issue the tile's products.  One thread spends about 560 clocks on a
// block of 64 along K (the wait for its operands, four tcgen05.mma, the commit), whatever the
// tile's width, while the tensor pipe needs 4 x 57 clocks for a width of 96 and 4 x 128 for 256
// (measured with operands resident in shared memory).  Narrow tiles are therefore issued by two
// threads of two warps: the first takes the even blocks of K into one accumulator, the second
// the odd ones into another, and the epilogue adds the two, always in that order.
template <int BN, int STAGES, bool PAIR, int ISSUERS>
__global__ void __launch_bounds__(THREADS + 32 * (ISSUERS - 1), 1)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_out, const GemmParams p, const int tiles_m, const int n_tiles) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int B_ROWS = PAIR ? BN / 2 : BN;             // rows of W this CTA loads per block of K
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = B_ROWS * BK * 2;
    constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;          // tokens per tile (of the pair)
    static_assert(ISSUERS == 1 || (ISSUERS == 2 && BN <= 128 && !PAIR), "two issuers: four accumulators of at most 128 columns");
    constexpr int ACC_STRIDE = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256), TMEM_COLS = 2 * ISSUERS * ACC_STRIDE, CHUNKS = BN / 32;
    unsigned char* stage_a = smem;
    unsigned char* stage_b = smem + STAGES * A_BYTES;
    float* turn_all = reinterpret_cast<float*>(smem + STAGES * (A_BYTES + B_BYTES));
    uint64_t* full = reinterpret_cast<uint64_t*>(turn_all + 8 * WARP_BLOCKS_BYTES / 4);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;        // [2]: the MMAs of a tile have finished
    uint64_t* acc_empty = acc_full + 2;         // [2]: the epilogue warps have read the tile out
    uint64_t* drained = acc_empty + 2;          // [2]: after a failure, an issuing thread's products have all finished
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drained + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_ok = reinterpret_cast<volatile int*>(tmem_slot + 2);     // [2], by the tile's parity
    // by the tile's parity, so that a warp may start on the next tile while another finishes this one:
    long* kv_off_all = reinterpret_cast<long*>(tmem_slot + 4);            // [2][128] element offset of each token in the cache pages
    float* bias_all = reinterpret_cast<float*>(kv_off_all + 2 * BM);      // [2][256] the tile's biases (zeros without a bias)

    dependents_may_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_k = (p.K + BK - 1) / BK;
    const bool stamps = p.timeline != nullptr && blockIdx.x == 0;
    if (stamps && threadIdx.x == 0) p.timeline[0] = now_ns();
    // A pair is the two CTAs of a cluster; it walks the tiles as one.
    const uint32_t rank = PAIR ? cluster_cta_rank() : 0u;
    const bool leader = rank == 0;
    const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], ISSUERS);            // one commit per issuing thread
            mbar_init(&acc_empty[a], PAIR ? 16 : 8);     // one arrival per epilogue warp (of both CTAs, at the leader)
            mbar_init(&drained[a], 1);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) tmem_alloc(tmem_slot, TMEM_COLS);
    tcgen05_before_sync();
    __syncthreads();
    if (PAIR) cluster_barrier();                 // the other CTA's barriers are initialised before anything arrives there
    tcgen05_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    auto give_up = [&](int code) {
        if (!*failed) {
            *failed = code;
            atomicExch(p.status, code);
        }
    };
    if (PAIR) {
        // An MMA of the pair writes the accumulator at one address in both CTAs' tensor
        // memories: the two allocations must have given the same one.
        if (threadIdx.x == 0 && load_u32_from_rank(tmem_slot, rank ^ 1u) != tmem_base) give_up(STATUS_PAIR_TMEM_DIFFERS);
        cluster_barrier();                       // both CTAs know before either starts
        if (threadIdx.x == 0 && leader && load_u32_from_rank(reinterpret_cast<const uint32_t*>(const_cast<const int*>(failed)), 1u) != 0u)
            give_up(STATUS_PAIR_TMEM_DIFFERS);
        __syncthreads();
    }

    wait_for_earlier_kernels();          // nothing above reads or writes the step's memory (the stamps are the caller's own)
    if (stamps && threadIdx.x == 0) p.timeline[1] = now_ns();
    // Each issuing thread has a ring of stages of its own (the first RING0 stages, the rest),
    // filled by the producer in the order in which that thread takes its blocks.  A stage that
    // two threads took in turn would let one of them look at a barrier two phases after it last
    // saw it, and a wait by parity cannot tell a phase from the one two before it.
    constexpr int RING0 = ISSUERS == 2 ? (STAGES + 1) / 2 : STAGES, RING1 = STAGES - RING0;
    static_assert(ISSUERS == 1 || RING1 >= 2, "two issuers: at least two stages each");
    if (warp == 8) {
        // ---- producer: the rings run on across tiles ----
        if (lane == 0) {
            int pos[2] = {0, 0};                     // the next stage of each ring
            uint32_t phase[2] = {0u, 0u};            // the parity of the round that stage is in
            int issued[2] = {0, 0};
            bool ok = true;
            for (int tile = walker; tile < n_tiles && ok && !*failed; tile += walkers) {
                const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
                for (int kb = 0; kb < num_k; kb++) {
                    const int ring = ISSUERS == 2 ? (kb & 1) : 0;
                    const int s = ring == 0 ? pos[0] : RING0 + pos[1];
                    if (!mbar_wait(&empty[s], phase[ring] ^ 1u) || *failed) {
                        give_up(STATUS_TIMEOUT_ROWS_PRODUCER);
                        ok = false;
                        break;
                    }
                    if (PAIR) {
                        // both CTAs' bytes count on the leader's barrier, which expects them all
                        const uint32_t bar = cluster_address_of(&full[s], 0);
                        if (leader) mbar_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));
                        tma_load_2d_pair(stage_a + s * A_BYTES, &map_a, bar, kb * BK, tile_m * TILE_ROWS + (int)rank * BM);
                        tma_load_2d_pair(stage_b + s * B_BYTES, &map_b, bar, kb * BK, tile_n * BN + (int)rank * B_ROWS);
                    } else {
                        mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                        tma_load_2d(stage_a + s * A_BYTES, &map_a, &full[s], kb * BK, tile_m * BM);
                        tma_load_2d(stage_b + s * B_BYTES, &map_b, &full[s], kb * BK, tile_n * BN);
                    }
                    issued[ring]++;
                    if (++pos[ring] == (ring == 0 ? RING0 : RING1)) {
                        pos[ring] = 0;
                        phase[ring] ^= 1u;
                    }
                }
            }
            if (*failed && leader) {
                // copies that were issued still land: wait for them (bounded) so that none is in flight at the end
                for (int ring = 0; ring < ISSUERS; ring++) {
                    const int size = ring == 0 ? RING0 : RING1;
                    for (int i = max(0, issued[ring] - size); i < issued[ring]; i++)
                        mbar_wait(&full[(ring == 0 ? 0 : RING0) + i % size], (uint32_t)(i / size) & 1u);
                }
            }
        }
    } else if (warp >= 9) {
        // ---- MMA issue: tile t into the accumulators of parity t % 2; issuer i takes the blocks
        // of K with kb % ISSUERS == i from its own ring.  The flag `failed` is looked at once a
        // tile: every other role's waits are bounded too, so a failure elsewhere ends this loop
        // by a wait running out.
        const int issuer = warp - 9;
        if (lane == 0 && leader) {
            // This thread's instructions between two blocks are what bounds the loop, so it keeps
            // the ring's position and the descriptors as running values.
            const uint32_t idesc = make_instr_desc(TILE_ROWS, BN);
            const int ring_base = issuer == 0 ? 0 : RING0, ring_size = issuer == 0 ? RING0 : RING1;
            // the address field counts 16 bytes and stays below its 14 bits for any stage
            const uint64_t desc_a0 = make_smem_desc(smem_u32(stage_a + ring_base * A_BYTES));
            const uint64_t desc_b0 = make_smem_desc(smem_u32(stage_b + ring_base * B_BYTES));
            uint64_t* const ring_full = full + ring_base;
            uint64_t* const ring_empty = empty + ring_base;
            int local = 0, pos = 0;
            uint32_t phase = 0u;
            long long looked = 0, not_there = 0;
            bool ok = true;
            for (int tile = walker; tile < n_tiles && ok && !*failed; tile += walkers, local++) {
                const int acc = local & 1;
                if (!mbar_wait(&acc_empty[acc], ((local >> 1) & 1) ^ 1) || *failed) {
                    give_up(STATUS_TIMEOUT_ROWS_MMA);
                    break;
                }
                tcgen05_after_sync();
                const uint32_t tmem_acc = tmem_base + (uint32_t)((acc * ISSUERS + issuer) * ACC_STRIDE);
                for (int kb = issuer; kb < num_k; kb += ISSUERS) {
                    looked++;
                    if (!mbar_try_wait(&ring_full[pos], phase)) {
                        not_there++;
                        if (!mbar_wait(&ring_full[pos], phase)) {
                            give_up(STATUS_TIMEOUT_ROWS_MMA);
                            ok = false;
                            break;
                        }
                    }
                    tcgen05_after_sync();
                    if (stamps && local == 0 && kb == 0) p.timeline[2] = now_ns();
                    const uint64_t desc_a = desc_a0 + (uint64_t)(pos * (A_BYTES >> 4));
                    const uint64_t desc_b = desc_b0 + (uint64_t)(pos * (B_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        if (PAIR) umma_pair(tmem_acc, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        else umma(tmem_acc, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb >= ISSUERS || k > 0) ? 1u : 0u);
                    }
                    if (PAIR) umma_commit_pair(&ring_empty[pos]);
                    else umma_commit(&ring_empty[pos]);
                    if (++pos == ring_size) {
                        pos = 0;
                        phase ^= 1u;
                    }
                }
                // (after a wait that ran out too: the epilogue is not left waiting for this thread)
                if (PAIR) umma_commit_pair(&acc_full[acc]);
                else umma_commit(&acc_full[acc]);
                if (stamps && local == 0 && issuer == 0) p.timeline[3] = now_ns();
            }
            if (stamps && issuer == 0) {
                p.timeline[7] = (unsigned long long)looked;
                p.timeline[8] = (unsigned long long)not_there;
            }
            if (*failed) {
                // products that were issued still run: wait for them (bounded) before the tensor memory is freed
                if (PAIR) umma_commit_pair(&drained[issuer]);
                else umma_commit(&drained[issuer]);
                mbar_wait(&drained[issuer], 0);
            }
        }
    } else {
        // ---- epilogue: warps w and w + 4 own TMEM lanes 32 (w % 4) .. +31 and take the tile's
        // blocks of 32 columns in turn ----
        const int quarter = warp & 3, col_half = warp >> 2;
        BlockOut out_ctx{&map_out, turn_all + warp * (WARP_BLOCKS_BYTES / 4), nullptr, nullptr, quarter, lane, 0};
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        int local = 0;
        for (int tile = walker; tile < n_tiles; tile += walkers, local++) {
            const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
            const int acc = local & 1;
            const int first_row = tile_m * TILE_ROWS + (int)rank * BM;      // this CTA's 128 tokens of the tile
            long* kv_off = kv_off_all + acc * BM;
            float* bias_s = bias_all + acc * 256;
            out_ctx.kv_off = kv_off;
            out_ctx.bias_s = bias_s;
            if (p.k_pages != nullptr && threadIdx.x < BM) {
                const int t = first_row + threadIdx.x;
                if (t < p.M) {
                    const int pos = p.positions[t];
                    const int page = p.block_table[(long)p.token_item[t] * p.max_blocks + pos / p.page_size];
                    kv_off[threadIdx.x] = ((long)page * p.page_size + pos % p.page_size) * p.kv_width;
                }
            }
            if (threadIdx.x < BN) {
                const int n = tile_n * BN + threadIdx.x;
                bias_s[threadIdx.x] = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.0f;
            }
            // One thread waits for the accumulator; all eight warps learn the outcome at one
            // barrier, so that they go on or leave together.
            if (threadIdx.x == 0) {
                const bool ok = mbar_wait(&acc_full[acc], (local >> 1) & 1) && !*failed;
                if (!ok) give_up(STATUS_TIMEOUT_ROWS_EPILOGUE);
                tile_ok[acc] = ok ? 1 : 0;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (tile_ok[acc] == 0) break;
            tcgen05_after_sync();
            if (stamps && local == 0 && threadIdx.x == 0) p.timeline[4] = now_ns();
            const int row0 = first_row + quarter * 32;
            const uint32_t acc_base = lane_base + (uint32_t)(acc * ISSUERS * ACC_STRIDE);
#pragma unroll 1
            for (int c = col_half; c < CHUNKS; c += 2) {
                const int c0 = c * 32, n0 = tile_n * BN + c0;
                if (n0 >= p.N) continue;
                float v[32];
                __syncwarp();
                tmem_load_32(acc_base + c0, v);
                if (ISSUERS == 2 && num_k > 1) {         // the second issuer's blocks (none when K has one block)
                    float odd[32];
                    tmem_load_32(acc_base + ACC_STRIDE + c0, odd);
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] += odd[i];
                }
                finish_block(out_ctx, p, map_out, v, c0, n0, row0);
            }
            // the accumulator may be overwritten once every warp has read its part
            tcgen05_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(cluster_address_of(&acc_empty[acc], 0));
                else mbar_arrive(&acc_empty[acc]);
            }
            if (stamps && local == 0 && threadIdx.x == 0) p.timeline[5] = now_ns();
        }
        if (lane == 0) bulk_wait_done();         // this warp's boxes have arrived before the kernel ends
    }

    tcgen05_before_sync();
    __syncthreads();
    if (PAIR) cluster_barrier();                 // neither CTA frees or leaves while the other may still use it
    if (stamps && threadIdx.x == 0) p.timeline[6] = now_ns();
    if (warp == 9) tmem_free(tmem_base, TMEM_COLS);
}

// ---- tiles of the rows orientation shared along K by the CTAs of a cluster ----------------
//
// A product with few output features and a long inner size (the second product of a
// feed-forward at a few thousand tokens) has too few wide tiles for the SMs, and with narrow
// tiles its main loop is bound by what the SMs can pull from L2.  Here the 2 to 4 CTAs of a
// cluster take one tile of 128 x BN together, each a share of the blocks of K into its own
// accumulator.  The tile's blocks of 32 columns number rank, rank + splits, ... are finished by
// the CTA of that rank: after a cluster barrier (every CTA is done with its stages, over which
// the exchanges lie) each CTA stores its partial sums of the other CTAs' blocks as fp32 into
// their shared memory (stores through distributed shared memory wait for no answer; loads
// would, once per block and rank) and arrives at their barriers; a CTA whose barrier is
// complete adds, for each of its blocks, the parts in the order of the ranks, its own from
// tensor memory and the others' from its shared memory, and sends the block on like the rows
// kernel does.  The sum of a block is therefore formed in one place in a fixed order.
// Wait (bounded) for a phase of a barrier at which other CTAs of the cluster arrive after
// storing into this CTA's shared memory: the acquire is at cluster scope.
__device__ __forceinline__ bool mbar_wait_parts(uint64_t* bar, uint32_t parity) {
    const unsigned long long start = now_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++) {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(smem_u32(bar)), "r"(parity)
                : "memory");
            if (ok) return true;
        }
        if (now_ns() - start > WAIT_LIMIT_NS) return false;
    }
}

enum { STATUS_TIMEOUT_SPLIT_PRODUCER = 16, STATUS_TIMEOUT_SPLIT_MMA = 17, STATUS_TIMEOUT_SPLIT_EPILOGUE = 18, STATUS_TIMEOUT_SPLIT_PARTS = 19 };

// Slots of 32 columns x 128 rows in a CTA's exchange: the blocks it finishes times the other CTAs'
// parts of each, for the number of CTAs (2 to 4) that needs the most.
__host__ __device__ constexpr int exchange_slots(int chunks) {
    int most = 0;
    for (int splits = 2; splits <= 4; splits++) {
        const int slots = (chunks + splits - 1) / splits * (splits - 1);
        most = slots > most ? slots : most;
    }
    return most;
}

template <int BN, int STAGES>
constexpr size_t rows_split_shared_bytes() {
    // stages (the exchange lies over them), the epilogue warps' turning blocks, barriers, words, biases
    constexpr size_t stages = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2), exchange = (size_t)exchange_slots(BN / 32) * BM * 128;
    return (stages > exchange ? stages : exchange) + 8 * WARP_BLOCKS_BYTES + (2 * STAGES + 4) * 8 + 16 + 256 * 4 + 1024;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_rows_split_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_out, const GemmParams p, const int tiles_m, const int splits) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, CHUNKS = BN / 32;
    constexpr size_t STAGE_BYTES = (size_t)STAGES * (A_BYTES + B_BYTES), EXCHANGE_BYTES = (size_t)exchange_slots(CHUNKS) * BM * 128;
    constexpr size_t FRONT = STAGE_BYTES > EXCHANGE_BYTES ? STAGE_BYTES : EXCHANGE_BYTES;
    unsigned char* stage_a = smem;
    unsigned char* stage_b = smem + STAGES * A_BYTES;
    float* turn_all = reinterpret_cast<float*>(smem + FRONT);
    uint64_t* full = reinterpret_cast<uint64_t*>(turn_all + 8 * WARP_BLOCKS_BYTES / 4);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* drained = acc_full + 1;
    uint64_t* parts_full = drained + 1;         // the other CTAs' parts of this CTA's blocks have arrived
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(parts_full + 2);     // (one slot left out: the biases below stay on a 16-byte boundary)
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_ok = reinterpret_cast<volatile int*>(tmem_slot + 2);
    float* bias_s = reinterpret_cast<float*>(tmem_slot + 4);              // [256] the tile's biases (zeros without a bias)

    dependents_may_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool stamps = p.timeline != nullptr && blockIdx.x == 0;
    if (stamps && threadIdx.x == 0) p.timeline[0] = now_ns();
    const int num_k = (p.K + BK - 1) / BK;
    const uint32_t rank = cluster_rank();
    const int tile = (int)blockIdx.x / splits;
    const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
    const int share = (num_k + splits - 1) / splits;
    const int kb_lo = min(num_k, (int)rank * share), kb_hi = min(num_k, kb_lo + share);
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(drained, 1);
        mbar_init(parts_full, 8 * (splits - 1));    // one arrival per epilogue warp of every other CTA
        *failed = 0;
        *tile_ok = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) tmem_alloc(tmem_slot, BN);
    tcgen05_before_sync();
    __syncthreads();
    tcgen05_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    auto give_up = [&](int code) {
        if (!*failed) {
            *failed = code;
            atomicExch(p.status, code);
        }
    };
    wait_for_earlier_kernels();
    if (stamps && threadIdx.x == 0) p.timeline[1] = now_ns();
    const uint32_t exchange = smem_u32(smem);        // [block of this CTA][other CTA][8 pieces of 4 columns][BM rows][4 floats]: a warp's rows lie side by side
    if (warp == 8) {
        if (lane == 0) {
            int issued = 0;
            for (int kb = kb_lo; kb < kb_hi; kb++) {
                const int i = kb - kb_lo, s = i % STAGES;
                if (!mbar_wait(&empty[s], (((uint32_t)(i / STAGES)) & 1u) ^ 1u) || *failed) {
                    give_up(STATUS_TIMEOUT_SPLIT_PRODUCER);
                    break;
                }
                mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                tma_load_2d(stage_a + s * A_BYTES, &map_a, &full[s], kb * BK, tile_m * BM);
                tma_load_2d(stage_b + s * B_BYTES, &map_b, &full[s], kb * BK, tile_n * BN);
                issued = i + 1;
            }
            if (*failed)       // copies that were issued still land: none may be in flight when the stages are written over
                for (int i = max(0, issued - STAGES); i < issued; i++) mbar_wait(&full[i % STAGES], (uint32_t)(i / STAGES) & 1u);
        }
    } else if (warp == 9) {
        if (lane == 0) {
            const uint32_t idesc = make_instr_desc(BM, BN);
            const uint64_t desc_a0 = make_smem_desc(smem_u32(stage_a)), desc_b0 = make_smem_desc(smem_u32(stage_b));
            for (int kb = kb_lo; kb < kb_hi; kb++) {
                const int i = kb - kb_lo, s = i % STAGES;
                if (!mbar_wait(&full[s], (uint32_t)(i / STAGES) & 1u)) {
                    give_up(STATUS_TIMEOUT_SPLIT_MMA);
                    break;
                }
                tcgen05_after_sync();
                if (stamps && i == 0) p.timeline[2] = now_ns();
                const uint64_t desc_a = desc_a0 + (uint64_t)(s * (A_BYTES >> 4)), desc_b = desc_b0 + (uint64_t)(s * (B_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) umma(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            umma_commit(acc_full);       // (after a wait that ran out too: the epilogue is not left waiting)
            if (stamps) p.timeline[3] = now_ns();
            if (*failed) {
                umma_commit(drained);
                mbar_wait(drained, 0);
            }
        }
    } else {
        if (threadIdx.x < BN) {
            const int n = tile_n * BN + threadIdx.x;
            bias_s[threadIdx.x] = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.0f;
        }
        if (threadIdx.x == 0) {
            const bool ok = mbar_wait(acc_full, 0) && !*failed;
            if (!ok) give_up(STATUS_TIMEOUT_SPLIT_EPILOGUE);
            *tile_ok = ok ? 1 : 0;
        }
    }
    // every CTA of the cluster is done with its stages (or has failed, and the step is lost anyway):
    // the exchanges, which lie over them, may be written
    tcgen05_before_sync();
    __syncthreads();
    cluster_sync();
    if (stamps && threadIdx.x == 0) p.timeline[4] = now_ns();
    const int owned = (CHUNKS + splits - 1) / splits;        // blocks of 32 columns a CTA finishes, at most
    if (warp < 8) {
        // ---- the parts of the blocks that other CTAs finish: tensor memory -> their exchanges ----
        const int quarter = warp & 3, col_half = warp >> 2;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int row = quarter * 32 + lane;
        if (*tile_ok) {
            tcgen05_after_sync();
#pragma unroll 1
            for (int c = col_half; c < CHUNKS; c += 2) {
                const int owner = c % splits;
                if (owner == (int)rank) continue;
                float v[32];
                if (kb_hi > kb_lo) {
                    tmem_load_32(lane_base + c * 32, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = 0.0f;       // no block of K fell to this CTA
                }
                // block c is the owner's block number c / splits; among its other CTAs this one is number `slot`
                const int slot = (int)rank < owner ? (int)rank : (int)rank - 1;
                const uint32_t local = exchange + (uint32_t)((((c / splits) * (splits - 1) + slot) * 8) * BM + row) * 16;
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)owner));
#pragma unroll
                for (int j = 0; j < 8; j++)
                    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote + j * (BM * 16)), "f"(v[4 * j]),
                                 "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                                 : "memory");
            }
        }
        // (a CTA that failed arrives too: the others are not left waiting, the status word says that the step is lost)
        __syncwarp();
        if (lane == 0)
            for (int other = 0; other < splits; other++)
                if (other != (int)rank) mbar_arrive_cluster(cluster_address_of(parts_full, (uint32_t)other));
        if (stamps && threadIdx.x == 0) p.timeline[5] = now_ns();
        // ---- this CTA's blocks: its own part from tensor memory, the others' from the exchange, in rank order ----
        // (waited for in any case: no CTA leaves while another may still store into its shared memory)
        const bool parts_there = mbar_wait_parts(parts_full, 0);
        if (!parts_there) give_up(STATUS_TIMEOUT_SPLIT_PARTS);
        if (*tile_ok && parts_there) {
            BlockOut out_ctx{&map_out, turn_all + warp * (WARP_BLOCKS_BYTES / 4), bias_s, nullptr, quarter, lane, 0};
            const int row0 = tile_m * BM + quarter * 32;
#pragma unroll 1
            for (int mine = col_half; mine < owned; mine += 2) {
                const int c = mine * splits + (int)rank;
                if (c >= CHUNKS) break;
                const int c0 = c * 32, n0 = tile_n * BN + c0;
                if (n0 >= p.N) continue;
                float v[32], own[32];
                if (kb_hi > kb_lo) {
                    tmem_load_32(lane_base + c0, own);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) own[i] = 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 32; i++) v[i] = 0.0f;
                for (int r = 0; r < splits; r++) {
                    if (r == (int)rank) {
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] += own[i];
                        continue;
                    }
                    const int slot = r < (int)rank ? r : r - 1;
                    const uint32_t src = exchange + (uint32_t)(((mine * (splits - 1) + slot) * 8) * BM + row) * 16;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float4 x = lds128(src + j * (BM * 16));
                        v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
                    }
                }
                finish_block(out_ctx, p, map_out, v, c0, n0, row0);
            }
            if (lane == 0) bulk_wait_done();     // this warp's boxes have arrived before the kernel ends
        }
    }
    // No CTA stores into another's shared memory after it has arrived there, and none reads
    // another's: a CTA may leave when it is done.
    tcgen05_before_sync();
    __syncthreads();
    if (stamps && threadIdx.x == 0) p.timeline[6] = now_ns();
    if (warp == 9) tmem_free(tmem_base, BN);
}

// ---- host side: tensor maps ------------------------------------------------------------

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled g_encode = nullptr;
std::mutex g_lock;

struct MapKey {
    const void* base;
    long rows, cols, ld;
    int box_rows;             // operands: rows of a box of 64 bf16 columns; results: -2 (bf16) or -4 (fp32), boxes of 32 x 32
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base);
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld;
        return h * 1000003u ^ (size_t)k.box_rows;
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

// A [rows, cols] bf16 matrix with row stride ld; boxes of box_rows x 64 elements, 128-byte
// swizzle, zero fill outside the matrix.
int tensor_map(const void* base, long rows, long cols, long ld, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_lock);
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result) != cudaSuccess ||
            fn == nullptr || result != cudaDriverEntryPointSuccess)
            return fail("gemm: the driver does not offer cuTensorMapEncodeTiled");
        g_encode = reinterpret_cast<EncodeTiled>(fn);
    }
    MapKey key{base, rows, cols, ld, box_rows};
    auto found = g_maps.find(key);
    if (found != g_maps.end()) {
        *out = found->second;
        return 0;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_error_text, MLLM_ERROR_BUFFER, "gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
        return 3;
    }
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, *out);
    return 0;
}

template <int BN, int STAGES>
int launch_swapped(const CUtensorMap& a, const CUtensorMap& b, const GemmParams& p, dim3 grid, cudaStream_t s) {
    constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16 + (BN > BM ? BN : BM) * 8 + 1024;   // barriers, TMEM slot, flag, ticket, cache offsets
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_swapped_kernel<BN, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("gemm: cannot raise the shared memory limit");
        configured = true;
    }
    if (grid.z > 1) {
        // the CTAs that share a tile along K form a cluster (they read each other's shared memory)
        return launched(launch_kernel_in_clusters(g_dependent_launch != 0, dim3(1, 1, grid.z), gemm_swapped_kernel<BN, STAGES>, grid,
                                                  dim3(THREADS), smem, s, a, b, p),
                        "gemm_swapped_kernel (clusters)");
    }
    return launched(launch_kernel(g_dependent_launch != 0, gemm_swapped_kernel<BN, STAGES>, grid, dim3(THREADS), smem, s, a, b, p),
                    "gemm_swapped_kernel");
}

// The map of a result [rows, cols] (bfloat16 or fp32, row stride ld elements) for boxes of 32
// rows x 32 columns, rows of 64 or 128 bytes in shared memory with the swizzle of that width.  Returns 1 (no error text) if the
// tensor is not laid out for TMA: a base or a row stride off 16-byte boundaries.
int output_map(const void* base, long rows, long cols, long ld, bool f32, CUtensorMap* out) {
    const int elem = f32 ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * elem) % 16 != 0 || g_encode == nullptr) return 1;
    std::lock_guard<std::mutex> guard(g_lock);
    MapKey key{base, rows, cols, ld, f32 ? -4 : -2};
    auto found = g_maps.find(key);
    if (found != g_maps.end()) {
        *out = found->second;
        return 0;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t step[2] = {1, 1};
    CUresult r = g_encode(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                          const_cast<void*>(base), dims, strides, box, step, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, *out);
    return 0;
}

template <int BN, int STAGES, bool PAIR, int ISSUERS = 1>
int launch_rows(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& o, const GemmParams& p, int sms,
                cudaStream_t s) {
    constexpr size_t smem = rows_shared_bytes<BN, STAGES, PAIR>();
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_rows_kernel<BN, STAGES, PAIR, ISSUERS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return fail("gemm: cannot raise the shared memory limit");
        configured = true;
    }
    const int tile_rows = PAIR ? 2 * BM : BM;
    const int tiles_m = (p.M + tile_rows - 1) / tile_rows, tiles_n = (p.N + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;
    if (!PAIR)
        return launched(launch_kernel(g_dependent_launch != 0, gemm_rows_kernel<BN, STAGES, PAIR, ISSUERS>, dim3(std::min(n_tiles, sms)),
                                      dim3(THREADS + 32 * (ISSUERS - 1)), smem, s, a, b, o, p, tiles_m, n_tiles),
                        "gemm_rows_kernel");
    // two CTAs per tile: a cluster of two
    return launched(launch_kernel_in_clusters(g_dependent_launch != 0, dim3(2, 1, 1), gemm_rows_kernel<BN, STAGES, PAIR, ISSUERS>,
                                              dim3(2 * std::min(n_tiles, sms / 2)), dim3(THREADS), smem, s, a, b, o, p, tiles_m,
                                              n_tiles),
                    "gemm_rows_kernel (pairs)");
}

template <int BN, int STAGES>
int launch_rows_split(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& o, const GemmParams& p, int splits,
                      cudaStream_t s) {
    constexpr size_t smem = rows_split_shared_bytes<BN, STAGES>();
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_rows_split_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
            return fail("gemm: cannot raise the shared memory limit");
        configured = true;
    }
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    return launched(launch_kernel_in_clusters(g_dependent_launch != 0, dim3(splits, 1, 1), gemm_rows_split_kernel<BN, STAGES>,
                                              dim3(splits * tiles_m * tiles_n), dim3(THREADS), smem, s, a, b, o, p, tiles_m, splits),
                    "gemm_rows_split_kernel");
}

}  // namespace

// The SM count of the current device (asked once per device).
static int sm_count() {
    static int counts[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (counts[device] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
        counts[device] = sms;
    }
    return counts[device];
}

// Whether the kernel takes a product: K a multiple of 8 (rows of both operands start on
// 16-byte boundaries) and 16-byte aligned bases and row strides.
extern "C" int mllm_gemm_takes(long K, long ldx, const void* x, const void* w) {
    return K > 0 && K % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(w) & 15) == 0;
}

// out[M, N] = epilogue(x[M, K] w[N, K]^T + bias).  x, w bf16 (K contiguous; x with row stride
// ldx); out bf16, or fp32 with out_f32 or the residual epilogue.  status: a device int that
// must be zero; a non-zero value afterwards means a bounded wait inside the kernel ran out.
// A product of few tokens and few tiles is split along K over the CTAs of a cluster, which add
// their partial sums through each other's shared memory in a fixed order.
struct GemmScatter {
    void* k_pages;
    void* v_pages;
    const int* positions;
    const int* token_item;
    const int* block_table;
    int max_blocks, page_size, q_width, kv_width;
};

// Tile width of the persistent kernel for a product of M x N x K: the width with the least
// estimated time.  Measured on a B200 (time stamps inside the kernel, GPT-2 small's four
// products): a block of 64 along K takes a CTA about 0.34 us at every width (0.35 us at 256,
// where the tensor pipe itself needs 0.28 us), so wide tiles do more per block; a product
// lasts as long as its busiest CTA, which walks ceil(tiles / SMs) tiles; epilogues run under
// the next tile's blocks except the last one, about 0.0105 us per column of the tile.
static int rows_tile_width(int M, int N, int K, int sms) {
    const int widths[5] = {256, 192, 128, 96, 64};
    const long tiles_m = (M + BM - 1) / BM, num_k = (K + BK - 1) / BK;
    int best = 128;
    double best_cost = -1.0;
    for (int i = 0; i < 5; i++) {
        const int bn = widths[i];
        if (bn > 64 && bn >= 2 * N) continue;                     // mostly padding
        const long tiles = tiles_m * ((N + bn - 1) / bn);
        const long rounds = (tiles + sms - 1) / sms;
        const double cost = (double)(rounds * num_k) * (bn > 192 ? 0.35 : 0.34) + 0.0105 * bn;
        if (best_cost < 0.0 || cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

// Whether tiles shared along K by clusters (gemm_rows_split_kernel) beat the persistent kernel's
// best width, and with which code (7000 + CTAs: tiles of 256 features; 7100 + CTAs: of 128); 0 if
// not.  Measured in replayed graphs: such a product takes 1.2 us + its share of the blocks of K
// (0.35 us each at 256 features, 0.30 at 128) + 9 us (5.5 at 128) for two cluster barriers, the
// exchange, the finishing and the launch of clusters; the persistent kernel 1.25 us + its blocks
// + its last epilogue.  Clusters of two fill the GPU; clusters of four were placed in one
// round at 120 CTAs and not at 144, and clusters of three not at 144 CTAs.
static int rows_split_code(int M, int N, int K, int sms, int width, bool scatter) {
    if (scatter) return 0;
    const long tiles_m = (M + BM - 1) / BM, num_k = (K + BK - 1) / BK;
    const long rounds = (tiles_m * ((N + width - 1) / width) + sms - 1) / sms;
    const double whole = 1.25 + (double)(rounds * num_k) * (width > 192 ? 0.35 : 0.34) + 0.0105 * width;
    int best = 0;
    double best_cost = 0.93 * whole;               // (not for less than the estimates are good for)
    for (int wide = 0; wide < 2; wide++) {
        const int bn = wide ? 256 : 128;
        if (bn >= 2 * N) continue;
        const long tiles = tiles_m * ((N + bn - 1) / bn);
        for (int splits = 2; splits <= 4; splits += 2) {
            if (tiles * splits > (splits == 2 ? sms : 13 * sms / 16) || num_k / splits < 4) continue;
            const double cost = 1.2 + (double)((num_k + splits - 1) / splits) * (wide ? 0.35 : 0.30) + (wide ? 9.0 : 5.5);
            if (cost < best_cost) {
                best_cost = cost;
                best = (wide ? 7000 : 7100) + splits;
            }
        }
    }
    return best;
}

static int gemm_bf16(void* out, const void* x, const void* w, const float* bias, int M, int N, int K, long ldx, long ldo,
                     int epilogue, int out_f32, int* status, const GemmScatter* scatter, void* stream, int forced_bn,
                     unsigned long long* timeline = nullptr) {
    if (M <= 0 || N <= 0) return 0;
    if (!mllm_gemm_takes(K, ldx, x, w)) return fail("gemm: K and the row stride of x must be multiples of 8, bases 16-byte aligned");
    if (epilogue == EPI_ADD && !out_f32) return fail("gemm: the residual sum is kept in 32-bit");
    if (status == nullptr) return fail("gemm: a status word is required");
    cudaStream_t s = (cudaStream_t)stream;
    GemmParams p{out, bias, status, M, N, K, ldo, epilogue, out_f32, 1,
                 nullptr, nullptr, nullptr, nullptr, nullptr, 0, 1, 0, 0, timeline, 0};
    if (scatter != nullptr) {
        if (out_f32 || epilogue != EPI_STORE) return fail("gemm: the scatter goes with a plain bfloat16 store");
        if (scatter->q_width % 32 != 0 || scatter->kv_width % 32 != 0 || scatter->q_width + 2 * scatter->kv_width != N ||
            scatter->page_size <= 0)
            return fail("gemm: the scatter needs query and key/value widths that are multiples of 32 and add up to N");
        p.k_pages = (bf16*)scatter->k_pages;
        p.v_pages = (bf16*)scatter->v_pages;
        p.positions = scatter->positions;
        p.token_item = scatter->token_item;
        p.block_table = scatter->block_table;
        p.max_blocks = scatter->max_blocks;
        p.page_size = scatter->page_size;
        p.q_width = scatter->q_width;
        p.kv_width = scatter->kv_width;
    }
    CUtensorMap map_x, map_w;
    const int sms = sm_count();
    // Which kernel: up to 64 tokens the one with swapped operands.  It also takes products of up
    // to 512 tokens with a long K and few output features (the feed-forward's second product in
    // steps of prompt portions): there the persistent kernel is one chain of K / 64 dependent
    // blocks on few CTAs (17 us at 768 x 3072 whatever the tokens), and tiles of 128 tokens
    // shared along K by a cluster take 8.4 to 11.4 us (measured at 128 to 512 tokens; from
    // 1,024 tokens on the persistent kernel is as fast or faster, as it is for a short K).
    // (A forced code 5000 + t: the kernel with swapped operands and tiles of t tokens.)
    const int blocks_of_k = (K + BK - 1) / BK;
    const bool long_k_few_tokens = M <= 512 && blocks_of_k >= 32 && scatter == nullptr &&
                                   (long)((N + BM - 1) / BM) * ((M + 127) / 128) * 2 <= sms;
    const bool swap = forced_bn == 0 ? M <= 64 || long_k_few_tokens : (forced_bn >= 5000 && forced_bn < 7000);
    if (!swap) {
        // a tile: 128 tokens x bn features on one CTA, or (code 1000 + bn) 256 tokens x bn on a pair of CTAs
        // (narrow tiles are issued by two threads: see gemm_rows_kernel)
        int code = forced_bn != 0 ? forced_bn : rows_tile_width(M, N, K, sms);
        if (forced_bn == 0) {
            const int split_code = rows_split_code(M, N, K, sms, code, scatter != nullptr);
            if (split_code != 0) code = split_code;
            else if (code <= 128) code += 2000;
        }
        if (code >= 7000) {
            // (code 7000 + s: tiles of 256 features shared along K by clusters of s CTAs; 7100 + s: tiles of 128)
            const int splits = code % 100, bn_split = code < 7100 ? 256 : 128;
            if (splits < 2 || splits > 4 || scatter != nullptr) return fail("gemm: tiles are shared along K by 2 to 4 CTAs, without scatter");
            int rc = tensor_map(x, M, K, ldx, BM, &map_x);
            if (rc) return rc;
            rc = tensor_map(w, N, K, K, bn_split, &map_w);
            if (rc) return rc;
            CUtensorMap map_out = map_x;
            p.out_by_tma = output_map(out, M, N, ldo, out_f32 != 0, &map_out) == 0;
            if (bn_split == 256) return launch_rows_split<256, 3>(map_x, map_w, map_out, p, splits, s);
            return launch_rows_split<128, 4>(map_x, map_w, map_out, p, splits, s);
        }
        const bool pair = code >= 1000 && code < 2000;
        const int bn = code % 1000;
        int rc = tensor_map(x, M, K, ldx, BM, &map_x);
        if (rc) return rc;
        rc = tensor_map(w, N, K, K, pair ? bn / 2 : bn, &map_w);
        if (rc) return rc;
        // results leave by TMA when `out` is laid out for it (with the scatter, out is [M, q_width])
        CUtensorMap map_out = map_x;
        p.out_by_tma = output_map(out, M, scatter != nullptr ? scatter->q_width : N, ldo, out_f32 != 0, &map_out) == 0;
        switch (code) {
        case 256: return launch_rows<256, 3, false>(map_x, map_w, map_out, p, sms, s);
        case 192: return launch_rows<192, 3, false>(map_x, map_w, map_out, p, sms, s);
        case 128: return launch_rows<128, 4, false>(map_x, map_w, map_out, p, sms, s);
        case 96: return launch_rows<96, 5, false>(map_x, map_w, map_out, p, sms, s);
        case 64: return launch_rows<64, 6, false>(map_x, map_w, map_out, p, sms, s);
        case 2128: return launch_rows<128, 4, false, 2>(map_x, map_w, map_out, p, sms, s);
        case 2096: return launch_rows<96, 5, false, 2>(map_x, map_w, map_out, p, sms, s);
        case 2064: return launch_rows<64, 6, false, 2>(map_x, map_w, map_out, p, sms, s);
        case 1256: return launch_rows<256, 4, true>(map_x, map_w, map_out, p, sms, s);
        case 1192: return launch_rows<192, 5, true>(map_x, map_w, map_out, p, sms, s);
        case 1128: return launch_rows<128, 6, true>(map_x, map_w, map_out, p, sms, s);
        case 1096: return launch_rows<96, 6, true>(map_x, map_w, map_out, p, sms, s);
        case 1064: return launch_rows<64, 6, true>(map_x, map_w, map_out, p, sms, s);
        default: return fail("gemm: the tile width is 64, 96, 128, 192 or 256 (1000 + width on pairs of CTAs, 2000 + width up to 128 with two issuing threads)");
        }
    }
    const int bn = forced_bn >= 5000 ? forced_bn - 5000 : (M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)));
    if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) return fail("gemm: tiles of 16, 32, 64, 128 or 256 tokens");
    int rc = tensor_map(x, M, K, ldx, bn, &map_x);
    if (rc) return rc;
    rc = tensor_map(w, N, K, K, BM, &map_w);
    if (rc) return rc;
    dim3 grid((N + BM - 1) / BM, (M + bn - 1) / bn);
    {
        // Few tiles: share each among a cluster of 8, 4 or 2 CTAs along K, so that more SMs
        // stream the weights (at least two k blocks per CTA)
        const int tiles = grid.x * grid.y, all_k = (K + BK - 1) / BK;
        for (int splits = 8; splits >= 2; splits /= 2)
            if (tiles * splits <= sms && all_k / splits >= 2) {
                p.splits = splits;
                grid.z = splits;
                break;
            }
    }
    // (many tiles, as for a vocabulary: fewer stages, so that two or three CTAs share an SM and
    // one's start and end fall under another's main loop)
    const bool many_tiles = (long)grid.x * grid.y > 2L * sms && p.splits <= 1;
    if (bn == 16) return many_tiles ? launch_swapped<16, 4>(map_w, map_x, p, grid, s) : launch_swapped<16, 8>(map_w, map_x, p, grid, s);
    if (bn == 32) return many_tiles ? launch_swapped<32, 4>(map_w, map_x, p, grid, s) : launch_swapped<32, 8>(map_w, map_x, p, grid, s);
    if (bn == 64 && many_tiles) return launch_swapped<64, 4>(map_w, map_x, p, grid, s);
    if (bn == 64) return launch_swapped<64, 8>(map_w, map_x, p, grid, s);
    if (bn == 128) return launch_swapped<128, 6>(map_w, map_x, p, grid, s);
    return launch_swapped<256, 4>(map_w, map_x, p, grid, s);
}

extern "C" int mllm_gemm_bf16(void* out, const void* x, const void* w, const float* bias, int M, int N, int K,
                              long ldx, long ldo, int epilogue, int out_f32, int* status, void* stream) {
    return gemm_bf16(out, x, w, bias, M, N, K, ldx, ldo, epilogue, out_f32, status, nullptr, stream, 0);
}

// The same through the persistent kernel with a given tile width (64, 96, 128, 192 or 256),
// whatever the number of rows: for tests, which run every width at sizes that leave tiles
// partly empty, and for measurements of the widths against each other.
extern "C" int mllm_gemm_bf16_tile(void* out, const void* x, const void* w, const float* bias, int M, int N, int K,
                                   long ldx, long ldo, int epilogue, int out_f32, int* status, int tile_width,
                                   unsigned long long* timeline, void* stream) {
    // 1000 + width: on a pair of CTAs; 2000 + width: two issuing threads (the launcher refuses what it has not)
    if (tile_width <= 0 || (tile_width >= 3000 && tile_width < 5000) || (tile_width > 5256 && tile_width < 7002) || tile_width > 7104)
        return fail("gemm: the tile width is 64, 96, 128, 192 or 256");
    return gemm_bf16(out, x, w, bias, M, N, K, ldx, ldo, epilogue, out_f32, status, nullptr, stream, tile_width, timeline);
}

// The fused query/key/value product of a layer: out [M, q_width] gets the queries; keys and
// values go straight to the slots of the cache pages [n_pages, page_size, kv_width] that each
// token's position and its request's row of the block table name.
extern "C" int mllm_gemm_bf16_qkv(void* out, const void* x, const void* w, const float* bias, int M, int N, int K,
                                  long ldx, long ldo, int* status, void* k_pages, void* v_pages, const int* positions,
                                  const int* token_item, const int* block_table, int max_blocks, int page_size,
                                  int q_width, int kv_width, void* stream) {
    GemmScatter scatter{k_pages, v_pages, positions, token_item, block_table, max_blocks, page_size, q_width, kv_width};
    return gemm_bf16(out, x, w, bias, M, N, K, ldx, ldo, EPI_STORE, 0, status, &scatter, stream, 0);
}
