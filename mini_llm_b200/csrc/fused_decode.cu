// One kernel for a whole decode step of a stack of pre-norm attention + dense feed-forward
// layers (bfloat16 weights, up to 16 tokens).
//
// A decode step of few tokens is a chain of ~60 tiny, dependent operations; launched as
// separate kernels each pays a launch gap and a cold start, which together cost an order of
// magnitude more than the step's memory traffic (the reference meets the same wall: 87
// launches per token, docs/kernels/007_fewer_launches.md:188).  Here one persistent CTA per
// SM walks the phases of every layer, separated by grid-wide barriers instead of kernel
// boundaries.  What a phase needs and what does not depend on the phase before it (its
// weight fragments, biases, norm gains, the values a residual sum adds to) is copied into
// shared memory asynchronously while the previous phase finishes and the grid synchronises;
// after the barrier only the activations remain to be read.
//
// Phases of a layer (every CTA takes an equal share of the 16-row blocks of each product):
//   1  q, k, v = LN1(hidden) W_qkv^T + b     k, v go straight into the cache pages
//   2  attention over the paged cache, one CTA per (token, head), its warps sharing the keys
//   3  hidden += attn W_o^T + b
//   4  up = act(LN2(hidden) W_fc^T + b)
//   5  hidden += up W_proj^T + b
// before them the embedding, after them the final norm on the wanted rows, the output head
// and the sampling candidates.  Products run on the tensor cores (mma.sync m16n8k16: the
// weights stream into the A fragments, up to sixteen tokens are the B fragments).
//
// The grid must be co-resident (cooperative launch).  Every barrier wait is bounded: a CTA
// that waits longer than the limit writes a status code; every CTA that sees the code set
// leaves the kernel.
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_fused)

struct FusedLayer {
    const float *ln1_g, *ln1_b;
    const bf16* w_qkv;
    const float* b_qkv;
    const bf16* w_o;
    const float* b_o;
    const float *ln2_g, *ln2_b;
    const bf16* w_fc;
    const float* b_fc;
    const bf16* w_proj;
    const float* b_proj;
    bf16* k_pages;
    bf16* v_pages;
    float score_scale, eps1, eps2;
    int activation;            // EPI_GELU_TANH or EPI_GELU_ERF
    int window;                // 0: all keys
};

struct FusedParams {
    const FusedLayer* layers;
    int n_layers;
    int E, H, Hkv, D, I, V;
    int T;                      // tokens of the step, one per entry
    const int* token_ids;
    const int* positions;
    const int* token_item;
    const int* block_table;
    int max_blocks, page_size;
    const int* want_rows;
    int n_want;
    const bf16* wte;
    const bf16* wpe;            // null: no learned positions
    const float *lnf_g, *lnf_b;
    float eps_f;
    const bf16* w_head;
    float* hidden;              // [T, E]
    bf16* q;                    // [T, H*D]
    bf16* attn;                 // [T, H*D]
    bf16* up;                   // [T, I]
    float* logits;              // [n_want, V]
    int sample;                 // 0: no sampling, 1: fill out_tokens
    const float* temperature;
    const float* top_p;
    const unsigned long long* seeds;
    const int* counters;
    int* out_tokens;
    int* kept;                  // null, or [n_kept]: the last sampled token of every request slot
    const int* want_slots;      // [n_want]: the slot a sampled row is kept for, or -1
    int n_kept;
    float* cand_value;          // [n_want, gridDim.x]
    int* cand_index;
    int* cand_done;             // one zeroed counter
    unsigned long long* barrier;    // monotonically increasing arrival counter
    int* status;
    unsigned long long* timeline;   // null, or room for 5 * layers + 3 time stamps
    int att_parts;                  // CTAs that share the keys of one (token, head): 1 .. 16
    float* att_partial;             // [T * H, att_parts, D + 2]: a part's output, maximum, sum
    int* att_counters;              // [T * H], zero between launches
    unsigned long long barrier_limit_ns;    // 0: the default limit of a barrier wait
    int skip_arrival;               // tests of the limit: CTA 0 does not arrive at the first barrier, so no CTA passes it
};

namespace {

constexpr int THREADS = 512;
constexpr int WARPS = THREADS / 32;
constexpr int MAX_TOKENS = 16;
constexpr int XS_PAD = 32;           // bf16 elements between the rows staged in shared memory
// RES (a template parameter of the kernel): K steps of weights a warp prefetches into shared
// memory per phase, 6, 4 or 2; the launcher takes the largest that leaves room for the staged
// activations (with one token tile of GPT-2 small there is room for every step of its widest
// product).
constexpr unsigned long long BARRIER_LIMIT_NS = 2000000000ull;
enum { OUT_BF16 = 0, OUT_ADD = 1, OUT_QKV = 2, OUT_LOGITS = 3 };

// One product phase, as data.
struct Phase {
    const bf16* w;             // [N, K]; null: no phase
    const float* bias;
    int N, K, kind;
    const float *gamma, *beta; // norm applied to the phase's input, or null
    int which;                 // 0 .. 3: the layer's products in their order, 4: the output head
};

struct Split;

// Regions of the dynamic shared memory.
struct Shared {
    bf16* xs;                  // staged activations [NT * 8][k_max + XS_PAD]
    float* red;                // partial tiles [WARPS][32][NT * 4]
    float* att;                // attention merge [WARPS][2 + 256]
    uint4* wbuf;               // prefetched weight fragments [2 * RES][THREADS]
    float* bias;               // [2][THREADS][2], by phase parity
    float* old;                // [THREADS][NT * 4]
    float* gb;                 // norm gain and shift [2][E]
    long* kv_base;             // [MAX_TOKENS] element offset of each token's slot in the pages
    int* pos;                  // [MAX_TOKENS]
    int* table;                // [T][max_blocks]
    const Split* splits;       // [5]: how each kind of product phase is split (the same in every layer)
};

__host__ __device__ inline size_t shared_bytes(int nt, int res, int E, int I, int HD, int max_blocks) {
    const int k_max = E > I ? (E > HD ? E : HD) : (I > HD ? I : HD);
    return (size_t)nt * 8 * (k_max + XS_PAD) * 2 + (size_t)WARPS * 32 * nt * 4 * 4 + (size_t)WARPS * (2 + 256) * 4 +
           (size_t)2 * res * THREADS * 16 + (size_t)2 * THREADS * 2 * 4 + (size_t)THREADS * nt * 4 * 4 +
           (size_t)2 * E * 4 + MAX_TOKENS * 8 + MAX_TOKENS * 4 + (size_t)MAX_TOKENS * max_blocks * 4 + 64;
}

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void copy_async_16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void copy_async_4(void* smem_dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
                 : "memory");
}

// Grid-wide barrier: release-add, then poll with acquire loads.  Returns false if the step
// has failed (limit hit here or elsewhere).  The counter only grows, by the grid's size per
// barrier; `target` (thread 0's, 0 before the first barrier) is the count that ends this
// barrier: the first one takes it from its ticket with a division, the others add to it.
__device__ bool grid_barrier(const FusedParams& p, unsigned long long& target) {
    __shared__ int ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        ok = 1;
        unsigned long long ticket;
        if (p.skip_arrival != 0 && blockIdx.x == 0 && target == 0)
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(ticket) : "l"(p.barrier) : "memory");
        else
            asm volatile("atom.add.release.gpu.global.u64 %0, [%1], 1;" : "=l"(ticket) : "l"(p.barrier) : "memory");
        target = target == 0 ? (ticket / gridDim.x + 1) * gridDim.x : target + gridDim.x;
        const unsigned long long limit = p.barrier_limit_ns != 0 ? p.barrier_limit_ns : BARRIER_LIMIT_NS;
        unsigned long long start = 0;
        for (unsigned spins = 0;; spins++) {
            unsigned long long seen;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(p.barrier) : "memory");
            if (seen >= target) break;
            if ((spins & 255u) == 255u) {
                if (start == 0) start = now_ns();
                int failed;
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(failed) : "l"(p.status) : "memory");
                if (failed != 0 || now_ns() - start > limit) {
                    if (failed == 0) atomicExch(p.status, 21);
                    ok = 0;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return ok != 0;
}

__device__ __forceinline__ void share_of(int n, int& first, int& count) {
    const int per = (n + gridDim.x - 1) / gridDim.x;
    first = blockIdx.x * per;
    count = max(0, min(n, first + per) - first);
}

// How a product phase is split over the CTA's warps (the same for prefetch and compute).
struct Split {
    int first, count;          // this CTA's 16-row blocks
    int split;                 // warps per block
    int blocks_at_a_time;      // blocks the CTA works on at a time
    int per_part;              // K steps (of 32) per warp
    int split_shift;           // log2(split)
};

__device__ __forceinline__ Split split_of(int N, int K, int kind) {
    Split s;
    share_of((N + 15) / 16, s.first, s.count);
    s.split = 1;
    s.blocks_at_a_time = WARPS;
    if (kind != OUT_LOGITS && s.count < WARPS) {
        int pow2 = 1;
        while (pow2 < s.count) pow2 *= 2;
        s.split = WARPS / pow2;
        s.blocks_at_a_time = pow2;
    }
    s.per_part = (K / 32 + s.split - 1) / s.split;
    s.split_shift = 31 - __clz(s.split);
    return s;
}

// Start copying what `phase` needs and what is final already: this thread's first weight
// fragments (its private slots of wbuf), the biases of its rows, the values its results are
// added to, and (all threads together) the gain and shift of the phase's input norm.
template <int NT, int RES, bool ADDS, bool NORMED>       // of `phase`: its results are added to hidden; its input is normed
__device__ void prefetch_phase(const FusedParams& p, const Shared& sm, const Phase& phase, int parity, int n_rows) {
    if (phase.w != nullptr) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int g = lane >> 2, q = lane & 3;
        const Split s = sm.splits[phase.which];
        const int b = warp >> s.split_shift, part = warp & (s.split - 1);
        if (b < s.count) {
            const int row_lo = (s.first + b) * 16 + g, row_hi = row_lo + 8;
            const bf16* w_lo = phase.w + (long)min(row_lo, phase.N - 1) * phase.K + q * 8;
            const bf16* w_hi = phase.w + (long)min(row_hi, phase.N - 1) * phase.K + q * 8;
            const int k_begin = part * s.per_part, k_end = min(phase.K / 32, k_begin + s.per_part);
            for (int u = 0; u < RES && k_begin + u < k_end; u++) {
                copy_async_16(sm.wbuf + (2 * u) * THREADS + threadIdx.x, w_lo + (k_begin + u) * 32);
                copy_async_16(sm.wbuf + (2 * u + 1) * THREADS + threadIdx.x, w_hi + (k_begin + u) * 32);
            }
            if (part == 0) {
                float* bias = sm.bias + (parity * THREADS + threadIdx.x) * 2;
                if (phase.bias != nullptr) {
                    if (row_lo < phase.N) copy_async_4(bias, phase.bias + row_lo);
                    if (row_hi < phase.N) copy_async_4(bias + 1, phase.bias + row_hi);
                }
                if (ADDS) {
#pragma unroll
                    for (int t = 0; t < NT; t++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int n = (i < 2) ? row_lo : row_hi, m = t * 8 + 2 * q + (i & 1);
                            if (n < phase.N && m < n_rows)
                                copy_async_4(sm.old + threadIdx.x * (NT * 4) + t * 4 + i, p.hidden + (long)m * phase.N + n);
                        }
                }
            }
        }
        if (NORMED) {
            for (int c = threadIdx.x; c < phase.K / 4; c += THREADS) {
                copy_async_16(sm.gb + c * 4, phase.gamma + c * 4);
                copy_async_16(sm.gb + phase.K + c * 4, phase.beta + c * 4);
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Stage rows of a bf16 matrix written earlier in this kernel (read through L2).  A thread
// takes the same 16 bytes of eight rows at a time: eight loads on their way and no division
// (an index taken apart by a run-time row length costs more than the copy).
template <int MT>
__device__ void stage_copy(bf16* xs, int K, const bf16* src, long ld_src, int n_rows) {
    const int ldx = K + XS_PAD, chunks = K / 8;
    for (int c = threadIdx.x; c < chunks; c += THREADS) {
#pragma unroll
        for (int m0 = 0; m0 < MT; m0 += 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                v[u] = make_uint4(0, 0, 0, 0);
                if (m0 + u < n_rows) v[u] = __ldcg(reinterpret_cast<const uint4*>(src + (long)(m0 + u) * ld_src + c * 8));
            }
#pragma unroll
            for (int u = 0; u < 8; u++) *reinterpret_cast<uint4*>(xs + (m0 + u) * ldx + c * 8) = v[u];
        }
    }
}

// Stage the layer norm of rows of the fp32 hidden state (gathered through `rows`, if given);
// gain and shift are in shared memory already.  One warp per row; the row is read once.
template <int MT>
__device__ void stage_norm(const FusedParams& p, bf16* xs, int K, const float* gb, float eps, const int* rows, int n_rows) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ldx = K + XS_PAD;
    constexpr int HELD = 8;                        // chunks of four values a lane keeps (rows up to 1024 wide)
    const int quads = K / 4;
    const bool held = quads <= 32 * HELD;
    for (int m = warp; m < MT; m += WARPS) {
        if (m >= n_rows) {
            for (int k = lane; k < K; k += 32) xs[m * ldx + k] = __float2bfloat16_rn(0.0f);
            continue;
        }
        const float4* row = reinterpret_cast<const float4*>(p.hidden + (long)(rows ? rows[m] : m) * K);
        float4 keep[HELD];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < HELD; i++) {
            keep[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (held && lane + 32 * i < quads) keep[i] = __ldcg(row + lane + 32 * i);
            sum += keep[i].x + keep[i].y + keep[i].z + keep[i].w;
        }
        if (!held)
            for (int qd = lane; qd < quads; qd += 32) {
                const float4 v = __ldcg(row + qd);
                sum += v.x + v.y + v.z + v.w;
            }
        const float mean = warp_sum(sum) / (float)K;
        float sq = 0.0f;
        if (held) {
#pragma unroll
            for (int i = 0; i < HELD; i++)
                if (lane + 32 * i < quads) {
                    const float a = keep[i].x - mean, b = keep[i].y - mean, c = keep[i].z - mean, d = keep[i].w - mean;
                    sq += a * a + b * b + c * c + d * d;
                }
        } else {
            for (int qd = lane; qd < quads; qd += 32) {
                const float4 v = __ldcg(row + qd);
                const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
                sq += a * a + b * b + c * c + d * d;
            }
        }
        const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + eps);
        auto emit = [&](int qd, const float4& v) {
            const float4 g = *reinterpret_cast<const float4*>(gb + qd * 4);
            const float4 b = *reinterpret_cast<const float4*>(gb + K + qd * 4);
            __nv_bfloat162 lo = __floats2bfloat162_rn((v.x - mean) * inv * g.x + b.x, (v.y - mean) * inv * g.y + b.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn((v.z - mean) * inv * g.z + b.z, (v.w - mean) * inv * g.w + b.w);
            *reinterpret_cast<uint2*>(xs + m * ldx + qd * 4) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        };
        if (held) {
#pragma unroll
            for (int i = 0; i < HELD; i++)
                if (lane + 32 * i < quads) emit(lane + 32 * i, keep[i]);
        } else {
            for (int qd = lane; qd < quads; qd += 32) emit(qd, __ldcg(row + qd));
        }
    }
}

// One m16n8k16 tensor-core product: D = A (16 x 16, weights) * B (16 x 8, activations) + D.
__device__ __forceinline__ void mma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Greedy rules: a NaN beats numbers, the lower index wins ties (engine/src/argmax.cu:8-18).
__device__ __forceinline__ bool better_candidate(float va, int ia, float vb, int ib) {
    const bool na = va != va, nb = vb != vb;
    if (ia < 0) return false;
    if (ib < 0) return true;
    if (na != nb) return na;
    if (na) return ia < ib;
    if (va != vb) return va > vb;
    return ia < ib;
}

// The sampling score of logit v of token m at vocabulary index n: the logit itself (greedy)
// or logit / T + Gumbel noise from the hash of (seed, counter, n), as in sampling_kernels.cu.
__device__ __forceinline__ float sampling_score(const FusedParams& p, int m, int n, float v) {
    const float temp = p.temperature ? p.temperature[m] : 0.0f;
    if (!(temp > 0.0f)) return v;
    const unsigned long long seed = p.seeds ? p.seeds[m] : 0ull;
    const unsigned counter = p.counters ? (unsigned)p.counters[m] : 0u;
    unsigned long long h = seed ^ ((unsigned long long)counter << 32);
    h += 0x9E3779B97F4A7C15ull; h = (h ^ (h >> 30)) * 0xBF58476D1CE4E5B9ull;
    h = (h ^ (h >> 27)) * 0x94D049BB133111EBull; h ^= h >> 31;
    h ^= (unsigned long long)n;
    h += 0x9E3779B97F4A7C15ull; h = (h ^ (h >> 30)) * 0xBF58476D1CE4E5B9ull;
    h = (h ^ (h >> 27)) * 0x94D049BB133111EBull; h ^= h >> 31;
    const float uni = ((float)(unsigned)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
    return v * (1.0f / temp) - logf(-logf(uni));
}

// One product phase on the tensor cores.  The CTA takes its share of the 16-row blocks of
// w [N, K]; with fewer blocks than warps, the warps of a block split its K range and their
// partial tiles meet in shared memory, added in part order.  The first RES K steps of a
// warp's first block were prefetched into wbuf; the rest stream in from L2 / HBM.
//
// A lane (g = lane / 4, q = lane % 4) takes eight consecutive K values of rows g and g + 8
// (16 bytes each) and the same eight K values of token g (16 bytes from shared memory).
// Which K value sits in which slot of the instruction does not matter to a sum as long as A
// and B agree, so the eight values feed two instructions: values 0..3 the first (slots 2q,
// 2q+1, 2q+8, 2q+9), values 4..7 the second.
// Once a thread has read its prefetched data it starts the prefetch of `next`.
// KIND is the phase's kind, NEXT_ADDS and NEXT_NORMED describe `next` (see prefetch_phase): known
// where the phase is called, so that each copy of this code holds one epilogue and one prefetch.
template <int NT, int RES, int KIND, bool NEXT_ADDS, bool NEXT_NORMED>
__device__ void product_phase(const FusedParams& p, const Shared& sm, const Phase& phase, int parity, int ldx, int n_rows,
                              int activation, const FusedLayer* layer, const Phase& next, float* best_value,
                              int* best_index) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int N = phase.N, K = phase.K;
    constexpr int kind = KIND;
    const Split sp = sm.splits[phase.which];
    const int split = sp.split, k_steps = K / 32;
    const bf16* xs = sm.xs;
    asm volatile("cp.async.wait_group 0;" ::: "memory");       // this thread's prefetched data has landed
    for (int b0 = 0; b0 < sp.count || b0 == 0; b0 += sp.blocks_at_a_time) {
        const int b = b0 + (warp >> sp.split_shift), part = warp & (split - 1);
        const bool active = b < sp.count;
        float acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; t++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[t][i] = 0.0f;
        const int row_lo = (sp.first + b) * 16 + g, row_hi = row_lo + 8;
        if (active) {
            // rows past N are read from the last row (their results are never stored)
            const bf16* w_lo = phase.w + (long)min(row_lo, N - 1) * K + q * 8;
            const bf16* w_hi = phase.w + (long)min(row_hi, N - 1) * K + q * 8;
            const bf16* x_lo = xs + g * ldx + q * 8;
            const int k_begin = part * sp.per_part, k_end = min(k_steps, k_begin + sp.per_part);
            int ks = k_begin;
            if (b0 == 0) {
                for (int u = 0; u < RES && ks < k_end; u++, ks++) {
                    const uint4 wl = sm.wbuf[(2 * u) * THREADS + threadIdx.x];
                    const uint4 wh = sm.wbuf[(2 * u + 1) * THREADS + threadIdx.x];
#pragma unroll
                    for (int t = 0; t < NT; t++) {
                        const uint4 xv = *reinterpret_cast<const uint4*>(x_lo + t * 8 * ldx + ks * 32);
                        mma_16816(acc[t], wl.x, wh.x, wl.y, wh.y, xv.x, xv.y);
                        mma_16816(acc[t], wl.z, wh.z, wl.w, wh.w, xv.z, xv.w);
                    }
                }
            }
            // The steps that were not prefetched stream in through a ring of four register
            // slots: a slot is used and asked for the step four further on at once, so that the
            // latency of a load is paid once per block and not once per four steps.
            uint4 wl[4], wh[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                wl[u] = make_uint4(0, 0, 0, 0);
                wh[u] = make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (ks + u < k_end) {
                    wl[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + (ks + u) * 32));
                    wh[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + (ks + u) * 32));
                }
            for (; ks < k_end; ks += 4) {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (ks + u < k_end) {
#pragma unroll
                        for (int t = 0; t < NT; t++) {
                            const uint4 xv = *reinterpret_cast<const uint4*>(x_lo + t * 8 * ldx + (ks + u) * 32);
                            mma_16816(acc[t], wl[u].x, wh[u].x, wl[u].y, wh[u].y, xv.x, xv.y);
                            mma_16816(acc[t], wl[u].z, wh[u].z, wl[u].w, wh[u].w, xv.z, xv.w);
                        }
                    }
                    if (ks + u + 4 < k_end) {
                        wl[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + (ks + u + 4) * 32));
                        wh[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + (ks + u + 4) * 32));
                    }
                }
            }
        }
        // Biases and the values to add to: prefetched for the warp's first block (read here,
        // before the next phase's replace them), fetched directly for any further block.
        float bias_lo = 0.0f, bias_hi = 0.0f, old[NT][4];
#pragma unroll
        for (int t = 0; t < NT; t++)
#pragma unroll
            for (int i = 0; i < 4; i++) old[t][i] = 0.0f;
        if (active && part == 0) {
            if (b0 == 0) {
                if (phase.bias != nullptr) {
                    bias_lo = sm.bias[(parity * THREADS + threadIdx.x) * 2];
                    bias_hi = sm.bias[(parity * THREADS + threadIdx.x) * 2 + 1];
                }
                if (kind == OUT_ADD) {
#pragma unroll
                    for (int t = 0; t < NT; t++)
#pragma unroll
                        for (int i = 0; i < 4; i++) old[t][i] = sm.old[threadIdx.x * (NT * 4) + t * 4 + i];
                }
            } else {
                if (phase.bias != nullptr) {
                    if (row_lo < N) bias_lo = __ldg(phase.bias + row_lo);
                    if (row_hi < N) bias_hi = __ldg(phase.bias + row_hi);
                }
                if (kind == OUT_ADD) {
#pragma unroll
                    for (int t = 0; t < NT; t++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int n = (i < 2) ? row_lo : row_hi, m = t * 8 + 2 * q + (i & 1);
                            if (n < N && m < n_rows) old[t][i] = __ldcg(p.hidden + (long)m * N + n);
                        }
                }
            }
        }
        if (b0 == 0) prefetch_phase<NT, RES, NEXT_ADDS, NEXT_NORMED>(p, sm, next, parity ^ 1, p.T);
        if (split > 1) {
            float* mine = sm.red + (warp * 32 + lane) * (NT * 4);
#pragma unroll
            for (int t = 0; t < NT; t++)
#pragma unroll
                for (int i = 0; i < 4; i++) mine[t * 4 + i] = acc[t][i];
            __syncthreads();
            if (active && part == 0) {
                for (int s = 1; s < split; s++) {
                    const float* other = sm.red + ((warp + s) * 32 + lane) * (NT * 4);
#pragma unroll
                    for (int t = 0; t < NT; t++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[t][i] += other[t * 4 + i];
                }
            }
            __syncthreads();
            if (part != 0) continue;
        }
        if (!active) continue;
        // accumulator i of tile t: row (g or g + 8), token t * 8 + 2q + (i & 1)
#pragma unroll
        for (int t = 0; t < NT; t++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int n = (i < 2) ? row_lo : row_hi;
                const int m = t * 8 + 2 * q + (i & 1);
                if (n >= N || m >= n_rows) continue;
                float v = acc[t][i] + ((i < 2) ? bias_lo : bias_hi);
                if (kind == OUT_ADD) {
                    p.hidden[(long)m * N + n] = old[t][i] + v;
                } else if (kind == OUT_BF16) {
                    if (activation == EPI_GELU_TANH) v = gelu_tanh_fast(v);
                    else if (activation == EPI_GELU_ERF) v = gelu_erf_f(v);
                    p.up[(long)m * N + n] = __float2bfloat16_rn(v);
                } else if (kind == OUT_QKV) {
                    const int q_width = p.H * p.D, kv_width = p.Hkv * p.D;
                    if (n < q_width) p.q[(long)m * q_width + n] = __float2bfloat16_rn(v);
                    else if (n < q_width + kv_width) layer->k_pages[sm.kv_base[m] + (n - q_width)] = __float2bfloat16_rn(v);
                    else layer->v_pages[sm.kv_base[m] + (n - q_width - kv_width)] = __float2bfloat16_rn(v);
                } else {
                    p.logits[(long)m * N + n] = v;
                    if (p.sample != 0) {
                        const float score = sampling_score(p, m, n, v);
                        const int slot = t * 2 + (i & 1);
                        if (better_candidate(score, n, best_value[slot], best_index[slot])) {
                            best_value[slot] = score;
                            best_index[slot] = n;
                        }
                    }
                }
            }
    }
}

// Phase 2: one CTA per (token, head) pair, or, when the pairs are so few that SMs would stay
// idle, p.att_parts CTAs per pair, each with a share of the keys.  A CTA's warps take its
// keys in turn (four keys and four values in flight per lane), each with an online softmax;
// the warps' states are merged through shared memory in warp order.  A pair in several parts
// is finished by the CTA that arrives last, which adds the parts in their order: nothing
// depends on timing.  (Measured: a part costs about 3 us for the hand-over, so parts pay only
// while every CTA has at most one.)
template <int D>
__device__ void attention_phase(const FusedParams& p, const Shared& sm, const FusedLayer& layer) {
    constexpr int LPK = D / 8, KPW = 32 / LPK, INFLIGHT = 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPK, group = lane / LPK;
    const int kv_width = p.Hkv * D;
    const int page_shift = (p.page_size & (p.page_size - 1)) == 0 ? 31 - __clz(p.page_size) : -1;
    float* sm_m = sm.att;                     // [WARPS]
    float* sm_l = sm.att + WARPS;             // [WARPS]
    float* sm_acc = sm.att + 2 * WARPS;       // [WARPS][D]
    __shared__ int last_part;
    const int parts = p.att_parts;
    for (int unit = blockIdx.x; unit < p.T * p.H * parts; unit += gridDim.x) {
        const int pair = unit / parts, part = unit % parts;
        const int h = pair % p.H, t = pair / p.H;
        const int pos = sm.pos[t];
        const int begin = (layer.window > 0 && pos - layer.window + 1 > 0) ? pos - layer.window + 1 : 0;
        // this part's keys: an equal share, in whole steps of a warp
        const int share = ((pos - begin + parts) / parts + KPW - 1) / KPW * KPW;
        const int first = begin + part * share, last = min(pos, first + share - 1);
        const int* bt = sm.table + t * p.max_blocks;
        const int hk = h / (p.H / p.Hkv);
        const uint4 q_raw = __ldcg(reinterpret_cast<const uint4*>(p.q + (long)t * p.H * D + (long)h * D + sub * 8));
        float m = -INFINITY, l = 0.0f;          // m in units of log2(e): an exponential is one instruction
        // The warp's keys in turn n = 0, 1, ...: key first + (n * WARPS + warp) * KPW + group.  A lane
        // keeps INFLIGHT keys and values on their way, one per slot; it takes the oldest, asks
        // for the key INFLIGHT turns later into the same slot and goes on to the next slot, so
        // loads, address arithmetic and the softmax update of different keys overlap.
        const int head_offset = hk * D + sub * 8;
        const int my_key = first + warp * KPW + group;
        uint4 kv[INFLIGHT], vv[INFLIGHT];
        // A turn past the end asks for the last key again (valid memory, never used): no lane
        // branches around its loads.
        const long v_from_k = layer.v_pages - layer.k_pages;
        auto ask = [&](uint4& k_slot, uint4& v_slot, int j) {
            j = min(j, last);
            // pages of a power of two are the rule: shift and mask instead of a division per key
            const int block = page_shift >= 0 ? j >> page_shift : j / p.page_size;
            const int within = page_shift >= 0 ? j & (p.page_size - 1) : j % p.page_size;
            const bf16* k_at = layer.k_pages + (((long)bt[block] * p.page_size + within) * kv_width + head_offset);
            k_slot = __ldcg(reinterpret_cast<const uint4*>(k_at));
            v_slot = __ldcg(reinterpret_cast<const uint4*>(k_at + v_from_k));
        };
#pragma unroll
        for (int s = 0; s < INFLIGHT; s++) ask(kv[s], vv[s], my_key + s * (WARPS * KPW));
        // the query is unpacked after the first keys are asked for: nothing waits for it before
        float qf[8], acc[8];
        unpack8(q_raw, qf);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            qf[i] *= layer.score_scale * 1.4426950408889634f;
            acc[i] = 0.0f;
        }
        for (int j0 = my_key; j0 - group <= last; j0 += INFLIGHT * WARPS * KPW) {
#pragma unroll
            for (int s = 0; s < INFLIGHT; s++) {
                const int j = j0 + s * (WARPS * KPW);
                float kf[8], vf[8];
                unpack8(kv[s], kf);
                unpack8(vv[s], vf);
                ask(kv[s], vv[s], j + INFLIGHT * (WARPS * KPW));
                float sc = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) sc = fmaf(qf[i], kf[i], sc);
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
                if (j <= last) {
                    const float m_new = fmaxf(m, sc);
                    const float corr = fast_exp2(m - m_new), e = fast_exp2(sc - m_new);
                    l = l * corr + e;
#pragma unroll
                    for (int i = 0; i < 8; i++) acc[i] = acc[i] * corr + e * vf[i];
                    m = m_new;
                }
            }
        }
        // merge the key groups of the warp (a butterfly over the group index)
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m, o), l_o = __shfl_xor_sync(0xffffffffu, l, o);
            const float big = fmaxf(m, m_o);
            const float wa = (m == -INFINITY) ? 0.0f : fast_exp2(m - big), wb = (m_o == -INFINITY) ? 0.0f : fast_exp2(m_o - big);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] = acc[i] * wa + __shfl_xor_sync(0xffffffffu, acc[i], o) * wb;
            l = l * wa + l_o * wb;
            m = big;
        }
        __syncthreads();                      // the scratch may still be read for the previous unit
        if (group == 0) {
#pragma unroll
            for (int i = 0; i < 8; i++) sm_acc[warp * D + sub * 8 + i] = acc[i];
        }
        if (lane == 0) {
            sm_m[warp] = m;
            sm_l[warp] = l;
        }
        __syncthreads();
        // R threads per output value, each over WARPS / R warps, then the R in a fixed order
        constexpr int R = (THREADS / D >= 4) ? 4 : THREADS / D;
        float top = -INFINITY, denom = 0.0f, o = 0.0f;
        if (threadIdx.x < R * D) {
            const int d = threadIdx.x / R, r = threadIdx.x % R;
            for (int w = r * (WARPS / R); w < (r + 1) * (WARPS / R); w++) top = fmaxf(top, sm_m[w]);
#pragma unroll
            for (int x = 1; x < R; x <<= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, x, R));
            for (int w = r * (WARPS / R); w < (r + 1) * (WARPS / R); w++) {
                const float weight = (sm_m[w] == -INFINITY) ? 0.0f : fast_exp2(sm_m[w] - top);
                denom += sm_l[w] * weight;
                o += sm_acc[w * D + d] * weight;
            }
#pragma unroll
            for (int x = 1; x < R; x <<= 1) {
                denom += __shfl_xor_sync(0xffffffffu, denom, x, R);
                o += __shfl_xor_sync(0xffffffffu, o, x, R);
            }
        }
        const bool writes = threadIdx.x < R * D && threadIdx.x % R == 0;
        const int out_d = threadIdx.x / R;
        bf16* out = p.attn + (long)t * p.H * D + (long)h * D;
        if (parts == 1) {
            if (writes) out[out_d] = __float2bfloat16_rn(o / denom);
            continue;
        }
        // leave this part's state; the part that arrives last finishes the pair
        float* mine = p.att_partial + ((long)pair * parts + part) * (D + 2);
        if (writes) {
            __stcg(mine + out_d, o);
            if (threadIdx.x == 0) {
                __stcg(mine + D, top);
                __stcg(mine + D + 1, denom);
            }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) last_part = atomicAdd(p.att_counters + pair, 1) == parts - 1;
        __syncthreads();
        if (last_part && threadIdx.x < D) {
            __threadfence();
            const float* all = p.att_partial + (long)pair * parts * (D + 2);
            float big = -INFINITY;
            for (int q = 0; q < parts; q++) big = fmaxf(big, __ldcg(all + q * (D + 2) + D));
            float sum = 0.0f, total = 0.0f;
            for (int q = 0; q < parts; q++) {
                const float mq = __ldcg(all + q * (D + 2) + D);
                const float weight = (mq == -INFINITY) ? 0.0f : fast_exp2(mq - big);
                sum += __ldcg(all + q * (D + 2) + threadIdx.x) * weight;
                total += __ldcg(all + q * (D + 2) + D + 1) * weight;
            }
            out[threadIdx.x] = __float2bfloat16_rn(sum / total);
            if (threadIdx.x == 0) p.att_counters[pair] = 0;      // ready for the next layer and launch
        }
    }
}

__device__ Phase phase_of(const FusedParams& p, int index) {
    Phase ph{nullptr, nullptr, 16, 32, OUT_BF16, nullptr, nullptr, 0};
    const int q_width = p.H * p.D, qkv_width = (p.H + 2 * p.Hkv) * p.D;
    if (index < 4 * p.n_layers) {
        const FusedLayer& layer = p.layers[index / 4];
        switch (index % 4) {
        case 0: ph = Phase{layer.w_qkv, layer.b_qkv, qkv_width, p.E, OUT_QKV, layer.ln1_g, layer.ln1_b, 0}; break;
        case 1: ph = Phase{layer.w_o, layer.b_o, p.E, q_width, OUT_ADD, nullptr, nullptr, 1}; break;
        case 2: ph = Phase{layer.w_fc, layer.b_fc, p.I, p.E, OUT_BF16, layer.ln2_g, layer.ln2_b, 2}; break;
        default: ph = Phase{layer.w_proj, layer.b_proj, p.E, p.I, OUT_ADD, nullptr, nullptr, 3}; break;
        }
    } else if (index == 4 * p.n_layers && p.n_want > 0) {
        ph = Phase{p.w_head, nullptr, p.V, p.E, OUT_LOGITS, p.lnf_g, p.lnf_b, 4};
    }
    return ph;
}

template <int NT, int RES>
__global__ void __launch_bounds__(THREADS, 1) fused_decode_kernel(const FusedParams p) {
    constexpr int MT = NT * 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int k_max = max(p.E, max(p.I, p.H * p.D));
    Shared sm;
    unsigned char* cursor = smem_raw;
    sm.xs = reinterpret_cast<bf16*>(cursor);      cursor += (size_t)MT * (k_max + XS_PAD) * 2;
    sm.red = reinterpret_cast<float*>(cursor);    cursor += (size_t)WARPS * 32 * NT * 4 * 4;
    sm.att = reinterpret_cast<float*>(cursor);    cursor += (size_t)WARPS * (2 + 256) * 4;
    sm.wbuf = reinterpret_cast<uint4*>(cursor);   cursor += (size_t)2 * RES * THREADS * 16;
    sm.bias = reinterpret_cast<float*>(cursor);   cursor += (size_t)2 * THREADS * 2 * 4;
    sm.old = reinterpret_cast<float*>(cursor);    cursor += (size_t)THREADS * NT * 4 * 4;
    sm.gb = reinterpret_cast<float*>(cursor);     cursor += (size_t)2 * p.E * 4;
    sm.kv_base = reinterpret_cast<long*>(cursor); cursor += MAX_TOKENS * 8;
    sm.pos = reinterpret_cast<int*>(cursor);      cursor += MAX_TOKENS * 4;
    sm.table = reinterpret_cast<int*>(cursor);
    // How each kind of phase is split over CTAs and warps: worked out once (it takes divisions).
    __shared__ Split splits[5];
    sm.splits = splits;
    if (threadIdx.x < 5) {
        const Phase ph = phase_of(p, threadIdx.x < 4 ? threadIdx.x : 4 * p.n_layers);
        splits[threadIdx.x] = split_of(ph.N, ph.K, ph.kind);
    }
    __syncthreads();

    int stamp = 0;
    unsigned long long barrier_target = 0;
    // timeline (may be null): CTA 0 notes the time after every phase, for profiling
    auto note = [&]() {
        if (p.timeline != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.timeline[stamp] = now_ns();
        stamp++;
    };
    note();
    float best_value[NT * 2];
    int best_index[NT * 2];
#pragma unroll
    for (int i = 0; i < NT * 2; i++) {
        best_value[i] = 0.0f;
        best_index[i] = -1;
    }

    // ---- the step's positions, block tables and cache slots, once ----
    for (int i = threadIdx.x; i < p.T * p.max_blocks; i += THREADS)
        sm.table[i] = p.block_table[(long)p.token_item[i / p.max_blocks] * p.max_blocks + i % p.max_blocks];
    if (threadIdx.x < p.T) {
        const int pos = p.positions[threadIdx.x];
        const int page = p.block_table[(long)p.token_item[threadIdx.x] * p.max_blocks + pos / p.page_size];
        sm.pos[threadIdx.x] = pos;
        sm.kv_base[threadIdx.x] = ((long)page * p.page_size + pos % p.page_size) * ((long)p.Hkv * p.D);
    }
    int index = 0;
    Phase phase = phase_of(p, 0);
    prefetch_phase<NT, RES, false, true>(p, sm, phase, 0, p.T);
    // ---- embedding: token t is written by CTA t % grid ----
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
        int token = p.token_ids[t];
        if (token < 0) {                 // "the token this request sampled last": still on the device
            const int slot = -1 - token;
            token = (p.kept != nullptr && slot < p.n_kept) ? __ldcg(p.kept + slot) : 0;
        }
        const long trow = (long)token * p.E, prow = p.wpe ? (long)p.positions[t] * p.E : 0;
        for (int c = threadIdx.x; c < p.E / 4; c += THREADS) {
            const uint2 tv = __ldg(reinterpret_cast<const uint2*>(p.wte + trow + c * 4));
            float4 v = make_float4(__uint_as_float(tv.x << 16), __uint_as_float(tv.x & 0xffff0000u),
                                   __uint_as_float(tv.y << 16), __uint_as_float(tv.y & 0xffff0000u));
            if (p.wpe) {
                const uint2 pv = __ldg(reinterpret_cast<const uint2*>(p.wpe + prow + c * 4));
                v.x += __uint_as_float(pv.x << 16); v.y += __uint_as_float(pv.x & 0xffff0000u);
                v.z += __uint_as_float(pv.y << 16); v.w += __uint_as_float(pv.y & 0xffff0000u);
            }
            reinterpret_cast<float4*>(p.hidden + (long)t * p.E)[c] = v;
        }
    }
    if (!grid_barrier(p, barrier_target)) return;
    note();

    for (int l = 0; l < p.n_layers; l++) {
        const FusedLayer& layer = p.layers[l];
        Phase next = phase_of(p, index + 1);
        // ---- phase 1 ----
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                  // gain and shift were copied by all threads
        stage_norm<MT>(p, sm.xs, p.E, sm.gb, layer.eps1, nullptr, p.T);
        __syncthreads();
        product_phase<NT, RES, OUT_QKV, true, false>(p, sm, phase, index & 1, p.E + XS_PAD, p.T, EPI_STORE, &layer, next, best_value,
                                                     best_index);
        if (!grid_barrier(p, barrier_target)) return;
        note();
        // ---- phase 2 ----
        switch (p.D) {
        case 16: attention_phase<16>(p, sm, layer); break;
        case 32: attention_phase<32>(p, sm, layer); break;
        case 64: attention_phase<64>(p, sm, layer); break;
        case 128: attention_phase<128>(p, sm, layer); break;
        default: attention_phase<256>(p, sm, layer); break;
        }
        if (!grid_barrier(p, barrier_target)) return;
        note();
        // ---- phase 3 ----
        phase = next; index++; next = phase_of(p, index + 1);
        stage_copy<MT>(sm.xs, phase.K, p.attn, phase.K, p.T);
        __syncthreads();
        product_phase<NT, RES, OUT_ADD, false, true>(p, sm, phase, index & 1, phase.K + XS_PAD, p.T, EPI_STORE, &layer, next,
                                                     best_value, best_index);
        if (!grid_barrier(p, barrier_target)) return;
        note();
        // ---- phase 4 ----
        phase = next; index++; next = phase_of(p, index + 1);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        stage_norm<MT>(p, sm.xs, p.E, sm.gb, layer.eps2, nullptr, p.T);
        __syncthreads();
        product_phase<NT, RES, OUT_BF16, true, false>(p, sm, phase, index & 1, p.E + XS_PAD, p.T, layer.activation, &layer, next,
                                                      best_value, best_index);
        if (!grid_barrier(p, barrier_target)) return;
        note();
        // ---- phase 5 ----
        phase = next; index++; next = phase_of(p, index + 1);
        stage_copy<MT>(sm.xs, p.I, p.up, p.I, p.T);
        __syncthreads();
        product_phase<NT, RES, OUT_ADD, false, true>(p, sm, phase, index & 1, p.I + XS_PAD, p.T, EPI_STORE, &layer, next, best_value,
                                                     best_index);
        if (!grid_barrier(p, barrier_target)) return;
        note();
        phase = next; index++;
    }
    if (p.n_want <= 0) return;

    // ---- final norm, head, sampling candidates ----
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    stage_norm<MT>(p, sm.xs, p.E, sm.gb, p.eps_f, p.want_rows, p.n_want);
    __syncthreads();
    product_phase<NT, RES, OUT_LOGITS, false, false>(p, sm, phase, index & 1, p.E + XS_PAD, p.n_want, EPI_STORE, nullptr,
                                                     phase_of(p, index + 1), best_value, best_index);
    note();
    if (p.sample == 0) return;
    // A lane holds candidates for tokens t*8 + 2q + j (slot t*2 + j): the lanes of equal q
    // compare theirs, then the warps through shared memory, then the CTAs (the CTA that
    // arrives last does that).
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < NT * 2; i++)
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_value[i], o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_index[i], o);
            if (better_candidate(ov, oi, best_value[i], best_index[i])) {
                best_value[i] = ov;
                best_index[i] = oi;
            }
        }
    __shared__ float cta_value[WARPS][MAX_TOKENS];
    __shared__ int cta_index[WARPS][MAX_TOKENS];
    __shared__ int is_last;
    if (lane < 4) {
#pragma unroll
        for (int i = 0; i < NT * 2; i++) {
            const int m = (i / 2) * 8 + 2 * lane + (i & 1);
            cta_value[warp][m] = best_value[i];
            cta_index[warp][m] = best_index[i];
        }
    }
    __syncthreads();
    if (threadIdx.x < p.n_want) {
        float v = 0.0f;
        int i = -1;
        for (int w = 0; w < WARPS; w++)
            if (better_candidate(cta_value[w][threadIdx.x], cta_index[w][threadIdx.x], v, i)) {
                v = cta_value[w][threadIdx.x];
                i = cta_index[w][threadIdx.x];
            }
        p.cand_value[(long)threadIdx.x * gridDim.x + blockIdx.x] = v;
        p.cand_index[(long)threadIdx.x * gridDim.x + blockIdx.x] = i;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(p.cand_done, 1);
        is_last = ticket == (int)gridDim.x - 1;
        if (is_last) *p.cand_done = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (warp < p.n_want) {
        float v = 0.0f;
        int i = -1;
        for (int c = lane; c < (int)gridDim.x; c += 32) {
            const float cv = __ldcg(p.cand_value + (long)warp * gridDim.x + c);
            const int ci = __ldcg(p.cand_index + (long)warp * gridDim.x + c);
            if (better_candidate(cv, ci, v, i)) { v = cv; i = ci; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, i, o);
            if (better_candidate(ov, oi, v, i)) { v = ov; i = oi; }
        }
        if (lane == 0) {
            p.out_tokens[warp] = i;
            if (p.kept != nullptr) {
                const int slot = p.want_slots[warp];
                if (slot >= 0 && slot < p.n_kept) p.kept[slot] = i;
            }
        }
    }
}

int g_sm_count = 0, g_smem_optin = 0;

template <int NT, int RES>
int launch(const FusedParams& p, size_t smem, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaFuncAttributes attributes;
        if (cudaFuncGetAttributes(&attributes, fused_decode_kernel<NT, RES>) != cudaSuccess ||
            cudaFuncSetAttribute(fused_decode_kernel<NT, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 g_smem_optin - (int)attributes.sharedSizeBytes) != cudaSuccess)
            return fail("fused_decode: cannot raise the shared memory limit");
        configured = true;
    }
    void* args[] = {const_cast<FusedParams*>(&p)};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(fused_decode_kernel<NT, RES>), dim3(g_sm_count),
                                                dim3(THREADS), args, smem, s);
    if (e != cudaSuccess) {
        snprintf(g_error_text, MLLM_ERROR_BUFFER, "fused_decode: cooperative launch failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return 2;
    }
    return check_launch("fused_decode_kernel");
}

}  // namespace

extern "C" int mllm_fused_layer_bytes(void) { return (int)sizeof(FusedLayer); }
extern "C" int mllm_fused_params_bytes(void) { return (int)sizeof(FusedParams); }

// Number of CTAs the step runs with (one per SM); sizes the candidate scratch.
extern "C" int mllm_fused_grid(void) {
    if (g_sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, device);
        cudaDeviceGetAttribute(&g_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    }
    return g_sm_count;
}

// The K steps of weights kept in shared memory: the most that fits beside everything else
// (0: nothing fits).
static int resident_steps(int T, int E, int I, int HD, int max_blocks) {
    const int nt = T <= 8 ? 1 : 2;
    for (int res = nt == 1 ? 6 : 4; res >= 2; res -= 2)
        if (shared_bytes(nt, res, E, I, HD, max_blocks) + 8 * 1024 <= (size_t)g_smem_optin) return res;
    return 0;
}

// Whether the kernel takes these sizes: up to 16 tokens, widths that are multiples of 32
// (one tensor-core step), a head size that is a power of two, and everything it keeps in
// shared memory fitting there.
extern "C" int mllm_fused_takes(int T, int E, int H, int Hkv, int D, int I, int max_blocks) {
    mllm_fused_grid();
    if (T < 1 || T > MAX_TOKENS) return 0;
    if (E % 32 != 0 || I % 32 != 0 || (H * D) % 32 != 0) return 0;
    if (!(D == 16 || D == 32 || D == 64 || D == 128 || D == 256)) return 0;
    if (Hkv <= 0 || H % Hkv != 0 || max_blocks <= 0) return 0;
    return resident_steps(T, E, I, H * D, max_blocks) > 0;
}

extern "C" int mllm_fused_decode_step(const FusedParams* params, void* stream) {
    const FusedParams& p = *params;
    if (!mllm_fused_takes(p.T, p.E, p.H, p.Hkv, p.D, p.I, p.max_blocks)) return fail("fused_decode: sizes not taken");
    if (p.n_want > p.T) return fail("fused_decode: more wanted rows than tokens");
    const int nt = p.T <= 8 ? 1 : 2, res = resident_steps(p.T, p.E, p.I, p.H * p.D, p.max_blocks);
    const size_t smem = shared_bytes(nt, res, p.E, p.I, p.H * p.D, p.max_blocks);
    cudaStream_t s = (cudaStream_t)stream;
    if (nt == 1) return res == 6 ? launch<1, 6>(p, smem, s) : (res == 4 ? launch<1, 4>(p, smem, s) : launch<1, 2>(p, smem, s));
    return res == 4 ? launch<2, 4>(p, smem, s) : launch<2, 2>(p, smem, s);
}
