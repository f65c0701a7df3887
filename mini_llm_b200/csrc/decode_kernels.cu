// Kernels for steps of few tokens (decoding, short prompt portions), bfloat16.
//
// With a handful of rows every matrix product is a stream of the weights
// through the SMs, bound by HBM bandwidth and by launch latency, as in the
// reference's batched matrix-vector kernel (engine/src/matvec_batch.cu:148-261:
// rows staged in shared memory, weights streamed once, bias / gelu / residual
// in the epilogue).  Here:
//
//   skinny_linear   out = epilogue(norm?(x) W^T + bias) for up to 16 rows per
//                   CTA; 16-byte weight loads, fp32 accumulation; optional
//                   layer-norm prologue (the norm never round-trips through
//                   memory), optional epilogue that scatters key and value
//                   columns straight into the cache pages.
//   layernorm       one warp per row, the row read once (the norm of long steps, and of
//                   steps whose products do not take the norm on the way in).
//   split_attention one CTA per (token, head, chunk of keys); partial softmax
//                   states go to scratch memory and the CTA that finishes
//                   last for its (token, head) merges them in chunk order, so
//                   the result does not depend on which CTA came last.
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_decode)

// ---------------------------------------------------------------------------
// skinny_linear
// ---------------------------------------------------------------------------
struct SkinnyParams {
    void* out;                 // bf16 [M, ldo] / fp32 [M, ldo] (EPI_ADD, or out_f32)
    const void* x;             // bf16 [M, ldx], or fp32 [*, K] with the norm prologue
    const bf16* w;             // [N, K], K contiguous
    const float* bias;         // [N] or null
    const float* gamma;        // norm prologue: gain and shift [K], else null
    const float* beta;
    const int* rows;           // norm prologue: source row of each output row, or null
    float eps;
    int M, N, K;
    long ldx, ldo;
    int epilogue;
    int out_f32;               // EPI_STORE into fp32 (logits)
    // scatter of key / value columns into pages (null k_pages: off)
    bf16* k_pages;
    bf16* v_pages;
    const int* positions;
    const int* token_item;
    const int* block_table;
    int max_blocks, page_size, q_width, kv_width;
};

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

template <int MT>      // rows of x per CTA (compile-time bound; M may be smaller)
__global__ void __launch_bounds__(256)
skinny_linear_kernel(const SkinnyParams p, int n_per_cta) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    dependents_may_start();
    wait_for_earlier_kernels();
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);            // [MT][K]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * MT;
    const int m_count = min(MT, p.M - m0);
    const int K = p.K;

    // ---- stage the rows of x (normalised first, if asked) as bf16 ----
    if (p.gamma != nullptr) {
        const float* src = reinterpret_cast<const float*>(p.x);
        for (int m = warp; m < MT; m += 8) {
            if (m < m_count) {
                const float* row = src + (long)(p.rows ? p.rows[m0 + m] : m0 + m) * K;
                float sum = 0.0f;
                for (int k = lane; k < K; k += 32) sum += row[k];
                float mean = warp_sum(sum) / (float)K;
                float sq = 0.0f;
                for (int k = lane; k < K; k += 32) {
                    float c = row[k] - mean;
                    sq += c * c;
                }
                float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + p.eps);
                for (int k = lane; k < K; k += 32)
                    xs[m * K + k] = __float2bfloat16_rn((row[k] - mean) * inv * p.gamma[k] + p.beta[k]);
            } else {
                for (int k = lane; k < K; k += 32) xs[m * K + k] = __float2bfloat16_rn(0.0f);
            }
        }
    } else {
        const bf16* src = reinterpret_cast<const bf16*>(p.x);
        const int chunks = K / 8;
        for (int i = threadIdx.x; i < MT * chunks; i += 256) {
            int m = i / chunks, c = i % chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < m_count) v = *reinterpret_cast<const uint4*>(src + (long)(m0 + m) * p.ldx + c * 8);
            *reinterpret_cast<uint4*>(xs + m * K + c * 8) = v;
        }
    }
    __syncthreads();

    const int n_begin = blockIdx.x * n_per_cta;
    const int n_end = min(p.N, n_begin + n_per_cta);
    const int chunks = K / 8;
    for (int n = n_begin + warp; n < n_end; n += 8) {
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0.0f;
        const bf16* wrow = p.w + (long)n * K;
        int c = lane;
        // two chunks in flight per lane
        for (; c + 32 < chunks; c += 64) {
            uint4 w0 = __ldg(reinterpret_cast<const uint4*>(wrow + c * 8));
            uint4 w1 = __ldg(reinterpret_cast<const uint4*>(wrow + (c + 32) * 8));
            float wf0[8], wf1[8];
            unpack8(w0, wf0);
            unpack8(w1, wf1);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float xf[8];
                unpack8(*reinterpret_cast<const uint4*>(xs + m * K + c * 8), xf);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[m] = fmaf(wf0[i], xf[i], acc[m]);
                unpack8(*reinterpret_cast<const uint4*>(xs + m * K + (c + 32) * 8), xf);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[m] = fmaf(wf1[i], xf[i], acc[m]);
            }
        }
        for (; c < chunks; c += 32) {
            uint4 w0 = __ldg(reinterpret_cast<const uint4*>(wrow + c * 8));
            float wf0[8];
            unpack8(w0, wf0);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float xf[8];
                unpack8(*reinterpret_cast<const uint4*>(xs + m * K + c * 8), xf);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[m] = fmaf(wf0[i], xf[i], acc[m]);
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = warp_sum(acc[m]);

        // lane m writes row m
        float mine = 0.0f;
#pragma unroll
        for (int m = 0; m < MT; m++)
            if (lane == m) mine = acc[m];
        if (lane < m_count) {
            const int row = m0 + lane;
            float v = mine + (p.bias ? p.bias[n] : 0.0f);
            if (p.epilogue == EPI_GELU_TANH) v = gelu_tanh_f(v);
            else if (p.epilogue == EPI_GELU_ERF) v = gelu_erf_f(v);
            if (p.k_pages != nullptr && n >= p.q_width) {
                int pos = p.positions[row];
                int page = p.block_table[(long)p.token_item[row] * p.max_blocks + pos / p.page_size];
                long slot = ((long)page * p.page_size + pos % p.page_size) * p.kv_width;
                if (n < p.q_width + p.kv_width) p.k_pages[slot + (n - p.q_width)] = __float2bfloat16_rn(v);
                else p.v_pages[slot + (n - p.q_width - p.kv_width)] = __float2bfloat16_rn(v);
            } else if (p.epilogue == EPI_ADD) {
                float* o = reinterpret_cast<float*>(p.out) + (long)row * p.ldo + n;
                *o += v;
            } else if (p.out_f32) {
                reinterpret_cast<float*>(p.out)[(long)row * p.ldo + n] = v;
            } else {
                reinterpret_cast<bf16*>(p.out)[(long)row * p.ldo + n] = __float2bfloat16_rn(v);
            }
        }
    }
}

static int g_smem_optin = -1;

template <int MT>
static int launch_skinny(const SkinnyParams& p, cudaStream_t s) {
    size_t smem = (size_t)MT * p.K * sizeof(bf16);
    if (g_smem_optin < 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    }
    if (smem > (size_t)g_smem_optin) return fail("skinny_linear: the rows do not fit shared memory");
    static size_t configured = 0;                 // per instantiation
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(skinny_linear_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             g_smem_optin);
        if (e != cudaSuccess) return fail("skinny_linear: cannot raise the shared memory limit");
        configured = g_smem_optin;
    }
    // columns per CTA: enough CTAs to fill the GPU, at least one column per warp
    int n_per_cta = p.N >= 8192 ? 32 : (p.N >= 2048 ? 16 : 8);
    dim3 grid((p.N + n_per_cta - 1) / n_per_cta, (p.M + MT - 1) / MT);
    return launched(launch_kernel(g_dependent_launch != 0, skinny_linear_kernel<MT>, grid, dim3(256), smem, s, p, n_per_cta),
                    "skinny_linear_kernel");
}

extern "C" int mllm_decode_skinny_linear(const SkinnyParams* params, void* stream) {
    const SkinnyParams& p = *params;
    if (p.M <= 0 || p.N <= 0) return 0;
    if (p.K <= 0 || p.K % 8 != 0) return fail("skinny_linear: K must be a positive multiple of 8");
    if (p.gamma == nullptr && p.ldx % 8 != 0) return fail("skinny_linear: the row stride of x must be a multiple of 8");
    if (p.epilogue == EPI_ADD && p.k_pages != nullptr) return fail("skinny_linear: no scatter with the residual sum");
    cudaStream_t s = (cudaStream_t)stream;
    if (p.M <= 1) return launch_skinny<1>(p, s);
    if (p.M <= 2) return launch_skinny<2>(p, s);
    if (p.M <= 4) return launch_skinny<4>(p, s);
    if (p.M <= 8) return launch_skinny<8>(p, s);
    return launch_skinny<16>(p, s);
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* global) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(global)
                 : "memory");
}

// ---------------------------------------------------------------------------
// split_attention
// ---------------------------------------------------------------------------
// Scratch layout (fp32): for every (token, head, chunk):
//   acc  [tokens, heads, max_chunks, head_size]   un-normalised weighted values
//   ml   [tokens, heads, max_chunks, 2]           running maximum, running sum
// and one int32 counter per (token, head), zero between launches.
template <int D>       // head size: 16, 32, 64, 128 or 256
__global__ void __launch_bounds__(128)
split_attention_kernel(bf16* __restrict__ out, long ld_out, const bf16* __restrict__ q, long ld_q,
                       const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                       const int* __restrict__ token_item, int n_heads, int n_kv_heads, int page_size, float scale,
                       int window, int chunk, int max_chunks, float* __restrict__ part_acc,
                       float* __restrict__ part_ml, int* __restrict__ counters) {
    constexpr int LPK = D / 8;             // lanes per key: each lane owns 8 of the head's dimensions
    constexpr int KPW = 32 / LPK;          // keys per warp per step
    dependents_may_start();
    wait_for_earlier_kernels();
    const int t = blockIdx.x, h = blockIdx.y, c = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPK, group = lane / LPK;
    const int p = positions[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int c_first = lo / chunk, c_last = p / chunk;
    if (c < c_first || c > c_last) return;
    const int begin = max(lo, c * chunk), end = min(p, c * chunk + chunk - 1);     // inclusive
    const int* bt = block_table + (long)token_item[t] * max_blocks;
    const int hk = h / (n_heads / n_kv_heads);
    const long kv_width = (long)n_kv_heads * D;

    float qf[8], acc[8];
    unpack8(*reinterpret_cast<const uint4*>(q + (long)t * ld_q + (long)h * D + sub * 8), qf);
    // scores are kept in units of log2(e): exp(x) = 2^(x log2 e) costs one instruction then
    const float scale_log2 = scale * 1.4426950408889634f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        qf[i] *= scale_log2;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;       // m in log2 units
    // Every lane of the warp runs the same trips (the shuffles need all of them); a lane
    // whose key lies past the end copies nothing and skips the update.  A trip brings two
    // keys and values per lane; RING trips are in flight per warp (cp.async into a ring in
    // shared memory that each lane reads back itself), so that a trip's latency (block table,
    // then the page) is paid once per chunk and not once per trip.
    constexpr int RING = 4;
    __shared__ uint4 ring[RING][2][2][128];       // [trip in flight][key of the lane][K, V][thread]
    const int first_key = begin + warp * KPW + group;
    const int trips = (end - (begin + warp * KPW)) / (8 * KPW) + 1;      // <= 0: nothing for this warp
    // pages of a power of two are the rule: shift and mask instead of a division per key
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const long head_offset = (long)hk * D + sub * 8;
    auto issue = [&](int trip) {
        if (trip < trips) {
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int j = first_key + trip * 8 * KPW + u * 4 * KPW;
                if (j <= end) {
                    const int block = page_shift >= 0 ? j >> page_shift : j / page_size;
                    const int within = page_shift >= 0 ? j & (page_size - 1) : j % page_size;
                    const long base = ((long)bt[block] * page_size + within) * kv_width + head_offset;
                    cp_async_16(&ring[trip % RING][u][0][threadIdx.x], k_pages + base);
                    cp_async_16(&ring[trip % RING][u][1][threadIdx.x], v_pages + base);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int i = 0; i < RING - 1; i++) issue(i);
    for (int trip = 0; trip < trips; trip++) {
        issue(trip + RING - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(RING - 1) : "memory");
        // the two keys of the trip share one rescaling of the running sums
        float sc[2], vf[2][8];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const bool valid = first_key + trip * 8 * KPW + u * 4 * KPW <= end;
            float kf[8];
            unpack8(ring[trip % RING][u][0][threadIdx.x], kf);
            unpack8(ring[trip % RING][u][1][threadIdx.x], vf[u]);
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) dot = fmaf(qf[i], kf[i], dot);
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            sc[u] = valid ? dot : -INFINITY;          // what an absent key left in the ring is never used
            if (!valid) {
#pragma unroll
                for (int i = 0; i < 8; i++) vf[u][i] = 0.0f;
            }
        }
        const float m_new = fmaxf(m, fmaxf(sc[0], sc[1]));
        if (m_new != -INFINITY) {
            const float corr = exp2f(m - m_new), e0 = exp2f(sc[0] - m_new), e1 = exp2f(sc[1] - m_new);
            l = fmaf(l, corr, e0 + e1);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] = fmaf(acc[i], corr, fmaf(e0, vf[0][i], e1 * vf[1][i]));
            m = m_new;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // merge the key groups of a warp, then the four warps, always in the same order
    __shared__ float sm_m[4][KPW];
    __shared__ float sm_l[4][KPW];
    __shared__ float sm_acc[4][KPW][D];
    if (sub == 0) {
        sm_m[warp][group] = m;
        sm_l[warp][group] = l;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) sm_acc[warp][group][sub * 8 + i] = acc[i];
    __syncthreads();
    float big = -INFINITY;
    for (int w = 0; w < 4; w++)
        for (int g = 0; g < KPW; g++) big = fmaxf(big, sm_m[w][g]);
    const long cell = (((long)t * n_heads + h) * max_chunks + c);
    for (int d = threadIdx.x; d < D; d += 128) {
        float o = 0.0f;
        for (int w = 0; w < 4; w++)
            for (int g = 0; g < KPW; g++) {
                float mg = sm_m[w][g];
                if (mg != -INFINITY) o += sm_acc[w][g][d] * exp2f(mg - big);
            }
        part_acc[cell * D + d] = o;
    }
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < 4; w++)
            for (int g = 0; g < KPW; g++) {
                float mg = sm_m[w][g];
                if (mg != -INFINITY) total += sm_l[w][g] * exp2f(mg - big);
            }
        part_ml[cell * 2] = big;
        part_ml[cell * 2 + 1] = total;
    }

    // the CTA that arrives last for this (token, head) merges the chunks
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int ticket = atomicAdd(&counters[t * n_heads + h], 1);
        is_last = (ticket == c_last - c_first);
        if (is_last) counters[t * n_heads + h] = 0;       // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const long first = ((long)t * n_heads + h) * max_chunks;
    float top = -INFINITY;
    for (int cc = c_first; cc <= c_last; cc++) top = fmaxf(top, __ldcg(part_ml + (first + cc) * 2));
    float denom = 0.0f;
    for (int cc = c_first; cc <= c_last; cc++)
        denom += __ldcg(part_ml + (first + cc) * 2 + 1) * exp2f(__ldcg(part_ml + (first + cc) * 2) - top);
    for (int d = threadIdx.x; d < D; d += 128) {
        float o = 0.0f;
        for (int cc = c_first; cc <= c_last; cc++)
            o += __ldcg(part_acc + (first + cc) * D + d) * exp2f(__ldcg(part_ml + (first + cc) * 2) - top);
        out[(long)t * ld_out + (long)h * D + d] = __float2bfloat16_rn(o / denom);
    }
}

extern "C" int mllm_decode_split_attention(void* out, long ld_out, const void* q, long ld_q, const void* k_pages,
                                           const void* v_pages, const int* block_table, int max_blocks,
                                           const int* positions, const int* token_item, int n_tokens, int n_heads,
                                           int n_kv_heads, int head_size, int page_size, float scale, int window,
                                           int chunk, int max_chunks, float* part_acc, float* part_ml, int* counters,
                                           void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        return fail("split_attention: heads must be a multiple of key/value heads");
    if (chunk <= 0 || max_chunks <= 0 || max_chunks > 65535 || n_heads > 65535)
        return fail("split_attention: bad chunking");
    if (ld_q % 8 != 0) return fail("split_attention: the row stride of q must be a multiple of 8");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, n_heads, max_chunks);
#define LAUNCH_SPLIT(D)                                                                                              \
    launch_kernel(g_dependent_launch != 0, split_attention_kernel<D>, grid, dim3(128), 0, s, (bf16*)out, ld_out,     \
                  (const bf16*)q, ld_q, (const bf16*)k_pages, (const bf16*)v_pages, block_table, max_blocks,         \
                  positions, token_item, n_heads, n_kv_heads, page_size, scale, window, chunk, max_chunks, part_acc, \
                  part_ml, counters)
    switch (head_size) {
    case 16: LAUNCH_SPLIT(16); break;
    case 32: LAUNCH_SPLIT(32); break;
    case 64: LAUNCH_SPLIT(64); break;
    case 128: LAUNCH_SPLIT(128); break;
    case 256: LAUNCH_SPLIT(256); break;
    default: return fail("split_attention: head size must be 16, 32, 64, 128 or 256");
    }
#undef LAUNCH_SPLIT
    return check_launch("split_attention_kernel");
}

// Whether split_attention takes a head size (the others run the plain kernel).
extern "C" int mllm_decode_split_attention_takes(int head_size) {
    return head_size == 16 || head_size == 32 || head_size == 64 || head_size == 128 || head_size == 256;
}

// ---------------------------------------------------------------------------
// group_attention: the same split-key attention with the products on mma.sync tiles.
//
// One CTA per (token, key/value head, chunk of keys); its four warps take tiles of 16 keys in
// turn.  The query heads that share the key/value head (1 to 8) are the rows of the tiles:
//   S[heads x 8 keys]  = Q[heads x dims] K^T      m16n8k16, A = Q (kept in registers), B = K
//   O[heads x 8 dims] += P[heads x 16 keys] V     A = P (the registers S came in), B = V
// Keys and values stream through a cp.async ring in shared memory (a warp's own slots); the
// key rows are read back as 16-byte chunks, the value tiles with ldmatrix.trans.  The dims of
// a row are taken in a permuted order that is the same for Q and K, so that a lane reads whole
// 16-byte chunks; both tiles are swizzled so that the reads have no bank conflicts.  The
// softmax is the online one of split_attention, per 16 keys, in 32-bit, in exp2 units; the
// partial states and their merge by the last CTA of a pair use split_attention's scratch
// layout.  Against one key per eight lanes this needs about a tenth of the instructions.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float& c0, float& c1, float& c2, float& c3, uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 two = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&two);
}

template <int D>       // head size: 64 or 128
__global__ void __launch_bounds__(128)
group_attention_kernel(bf16* __restrict__ out, long ld_out, const bf16* __restrict__ q, long ld_q,
                       const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                       const int* __restrict__ token_item, int n_heads, int n_kv_heads, int page_size, float scale,
                       int window, int chunk, int max_chunks, float* __restrict__ part_acc,
                       float* __restrict__ part_ml, int* __restrict__ counters) {
    constexpr int CH = D / 8;              // 16-byte chunks of a key or value row
    constexpr int PAIRS = D / 32;          // chunks a lane reads of a key row (each serves two k steps)
    constexpr int NT = D / 8;              // 8-dim tiles of the output
    constexpr int RING = 256 / D;          // tiles of 16 keys in flight per warp: 4 (D = 64) or 2
    constexpr int TILE_BYTES = 16 * D * 2; // one tile of keys (or values)
    extern __shared__ __align__(16) unsigned char ga_smem[];
    dependents_may_start();
    wait_for_earlier_kernels();
    const int t = blockIdx.x, hk = blockIdx.y, c = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int heads = n_heads / n_kv_heads;            // 1..8: rows of the tiles
    const int p = positions[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int c_first = lo / chunk, c_last = p / chunk;
    if (c < c_first || c > c_last) return;
    const int begin = max(lo, c * chunk), end = min(p, c * chunk + chunk - 1);     // inclusive
    const int* bt = block_table + (long)token_item[t] * max_blocks;
    const long kv_width = (long)n_kv_heads * D;
    const float scale_log2 = scale * 1.4426950408889634f;
    unsigned char* ring_k = ga_smem + (size_t)warp * RING * 2 * TILE_BYTES;
    unsigned char* ring_v = ring_k + RING * TILE_BYTES;

    // the queries of this lane's row: chunk 4u + tq serves k steps 2u (words 0, 1) and 2u + 1 (words 2, 3)
    uint32_t qa[PAIRS][4];
#pragma unroll
    for (int u = 0; u < PAIRS; u++) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < heads) v = *reinterpret_cast<const uint4*>(q + (long)t * ld_q + (long)(hk * heads + g) * D + (4 * u + tq) * 8);
        qa[u][0] = v.x; qa[u][1] = v.y; qa[u][2] = v.z; qa[u][3] = v.w;
    }
    float o[NT][2];
#pragma unroll
    for (int j = 0; j < NT; j++) o[j][0] = o[j][1] = 0.0f;
    float m = -INFINITY, l = 0.0f;         // of row g; l is this lane's share of the sum

    const int n_tiles = (end - begin) / 16 + 1;                         // of the chunk
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + 3) / 4 : 0; // tiles warp, warp + 4, ...
    auto issue = [&](int i) {
        if (i < my_tiles) {
            const int first = begin + (warp + 4 * i) * 16;
            unsigned char* tk = ring_k + (i % RING) * TILE_BYTES;
            unsigned char* tv = ring_v + (i % RING) * TILE_BYTES;
#pragma unroll
            for (int r = 0; r < CH / 2; r++) {
                const int idx = lane + 32 * r, key = idx / CH, ch = idx % CH;
                const int j = first + key;
                // keys: chunk position xor 4 on odd rows; values: xor the row's low three bits
                unsigned char* dk = tk + key * (D * 2) + ((ch & ~7) | ((ch ^ ((key & 1) << 2)) & 7)) * 16;
                unsigned char* dv = tv + key * (D * 2) + ((ch & ~7) | ((ch ^ key) & 7)) * 16;
                if (j <= end) {
                    const long base = ((long)bt[j / page_size] * page_size + (j % page_size)) * kv_width + (long)hk * D + ch * 8;
                    cp_async_16(dk, k_pages + base);
                    cp_async_16(dv, v_pages + base);
                } else {
                    *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);     // a value that is never weighted must not be NaN
                    *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int i = 0; i < RING - 1; i++) issue(i);
    for (int i = 0; i < my_tiles; i++) {
        issue(i + RING - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(RING - 1) : "memory");
        __syncwarp();                                   // every lane's copies of this tile have landed
        const int first = begin + (warp + 4 * i) * 16;
        const unsigned char* tk = ring_k + (i % RING) * TILE_BYTES;
        const uint32_t tv = (uint32_t)__cvta_generic_to_shared(ring_v + (i % RING) * TILE_BYTES);
        // scores of row g against keys 2 tq, 2 tq + 1 of both halves of the tile
        float s[2][4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            s[h][0] = s[h][1] = s[h][2] = s[h][3] = 0.0f;
            const int key = 8 * h + g;
#pragma unroll
            for (int u = 0; u < PAIRS; u++) {
                const int ch = 4 * u + tq;
                const uint4 kb = *reinterpret_cast<const uint4*>(tk + key * (D * 2) + ((ch & ~7) | ((ch ^ ((key & 1) << 2)) & 7)) * 16);
                mma_bf16_16816(s[h][0], s[h][1], s[h][2], s[h][3], qa[u][0], 0u, qa[u][1], 0u, kb.x, kb.y);
                mma_bf16_16816(s[h][0], s[h][1], s[h][2], s[h][3], qa[u][2], 0u, qa[u][3], 0u, kb.z, kb.w);
            }
        }
        float tile_max = -INFINITY;
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int j = first + 8 * h + 2 * tq + e;
                s[h][e] = j <= end ? s[h][e] * scale_log2 : -INFINITY;
                tile_max = fmaxf(tile_max, s[h][e]);
            }
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
        const float m_new = fmaxf(m, tile_max);           // finite: the tile's first key is never past the end
        const float corr = exp2f(m - m_new);
        const float p00 = exp2f(s[0][0] - m_new), p01 = exp2f(s[0][1] - m_new);
        const float p10 = exp2f(s[1][0] - m_new), p11 = exp2f(s[1][1] - m_new);
        const uint32_t pa0 = pack_bf16(p00, p01), pa1 = pack_bf16(p10, p11);
        // the sum uses the rounded weights the product below sees
        const __nv_bfloat162 r0 = *reinterpret_cast<const __nv_bfloat162*>(&pa0), r1 = *reinterpret_cast<const __nv_bfloat162*>(&pa1);
        l = l * corr + (__low2float(r0) + __high2float(r0)) + (__low2float(r1) + __high2float(r1));
        m = m_new;
        float unused0 = 0.0f, unused1 = 0.0f;             // rows 8..15 of the tiles
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
            // four 8 x 8 blocks of the value tile, transposed: (keys 0-7 | 8-15) x (dims 8j.. | 8(j+1)..)
            const int key = (lane & 7) + ((lane >> 3) & 1) * 8, ch = j + (lane >> 4);
            uint32_t b0, b1, b2, b3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                         : "r"(tv + key * (D * 2) + ((ch & ~7) | ((ch ^ key) & 7)) * 16));
            o[j][0] *= corr; o[j][1] *= corr; o[j + 1][0] *= corr; o[j + 1][1] *= corr;
            mma_bf16_16816(o[j][0], o[j][1], unused0, unused1, pa0, 0u, pa1, 0u, b0, b1);
            mma_bf16_16816(o[j + 1][0], o[j + 1][1], unused0, unused1, pa0, 0u, pa1, 0u, b2, b3);
        }
        __syncwarp();                                   // the slot is copied into again two issues from now
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);

    // merge the four warps (through the ring, free by now), always in the same order
    __syncthreads();
    float* sm_m = reinterpret_cast<float*>(ga_smem);           // [4][8]
    float* sm_l = sm_m + 32;                                   // [4][8]
    float* sm_acc = sm_l + 32;                                 // [4][8][D]
    if (tq == 0) {
        sm_m[warp * 8 + g] = m;
        sm_l[warp * 8 + g] = l;
    }
#pragma unroll
    for (int j = 0; j < NT; j++) {
        sm_acc[(warp * 8 + g) * D + 8 * j + 2 * tq] = o[j][0];
        sm_acc[(warp * 8 + g) * D + 8 * j + 2 * tq + 1] = o[j][1];
    }
    __syncthreads();
    __shared__ int is_last[8];
    for (int row = 0; row < heads; row++) {
        const int h = hk * heads + row;
        float big = -INFINITY;
        for (int w = 0; w < 4; w++) big = fmaxf(big, sm_m[w * 8 + row]);
        const long cell = (((long)t * n_heads + h) * max_chunks + c);
        for (int d = threadIdx.x; d < D; d += 128) {
            float acc = 0.0f;
            for (int w = 0; w < 4; w++) {
                const float mw = sm_m[w * 8 + row];
                if (mw != -INFINITY) acc += sm_acc[(w * 8 + row) * D + d] * exp2f(mw - big);
            }
            part_acc[cell * D + d] = acc;
        }
        if (threadIdx.x == 0) {
            float total = 0.0f;
            for (int w = 0; w < 4; w++) {
                const float mw = sm_m[w * 8 + row];
                if (mw != -INFINITY) total += sm_l[w * 8 + row] * exp2f(mw - big);
            }
            part_ml[cell * 2] = big;
            part_ml[cell * 2 + 1] = total;
        }
    }
    // the CTA that arrives last for a (token, head) merges the chunks
    __threadfence();
    __syncthreads();
    if (threadIdx.x < heads) {
        const int h = hk * heads + threadIdx.x;
        const int ticket = atomicAdd(&counters[t * n_heads + h], 1);
        is_last[threadIdx.x] = (ticket == c_last - c_first);
        if (is_last[threadIdx.x]) counters[t * n_heads + h] = 0;      // ready for the next launch
    }
    __syncthreads();
    for (int row = 0; row < heads; row++) {
        if (!is_last[row]) continue;
        __threadfence();
        const int h = hk * heads + row;
        const long first_cell = ((long)t * n_heads + h) * max_chunks;
        float top = -INFINITY;
        for (int cc = c_first; cc <= c_last; cc++) top = fmaxf(top, __ldcg(part_ml + (first_cell + cc) * 2));
        float denom = 0.0f;
        for (int cc = c_first; cc <= c_last; cc++)
            denom += __ldcg(part_ml + (first_cell + cc) * 2 + 1) * exp2f(__ldcg(part_ml + (first_cell + cc) * 2) - top);
        for (int d = threadIdx.x; d < D; d += 128) {
            float acc = 0.0f;
            for (int cc = c_first; cc <= c_last; cc++)
                acc += __ldcg(part_acc + (first_cell + cc) * D + d) * exp2f(__ldcg(part_ml + (first_cell + cc) * 2) - top);
            out[(long)t * ld_out + (long)h * D + d] = __float2bfloat16_rn(acc / denom);
        }
    }
}

// Whether group_attention takes a layout: head size 64 or 128, at most eight query heads per
// key/value head, rows of q on 16-byte boundaries.
extern "C" int mllm_decode_group_attention_takes(int head_size, int n_heads, int n_kv_heads, long ld_q, const void* q) {
    return (head_size == 64 || head_size == 128) && n_kv_heads > 0 && n_heads % n_kv_heads == 0 &&
           n_heads / n_kv_heads <= 8 && ld_q % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0;
}

// Same arguments and scratch as mllm_decode_split_attention; chunk must be a multiple of 16.
extern "C" int mllm_decode_group_attention(void* out, long ld_out, const void* q, long ld_q, const void* k_pages,
                                           const void* v_pages, const int* block_table, int max_blocks,
                                           const int* positions, const int* token_item, int n_tokens, int n_heads,
                                           int n_kv_heads, int head_size, int page_size, float scale, int window,
                                           int chunk, int max_chunks, float* part_acc, float* part_ml, int* counters,
                                           void* stream) {
    if (n_tokens <= 0) return 0;
    if (!mllm_decode_group_attention_takes(head_size, n_heads, n_kv_heads, ld_q, q))
        return fail("group_attention: head size 64 or 128, at most 8 query heads per key/value head, q 16-byte aligned");
    if (chunk <= 0 || chunk % 16 != 0 || max_chunks <= 0 || max_chunks > 65535 || n_kv_heads > 65535)
        return fail("group_attention: bad chunking");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, n_kv_heads, max_chunks);
    const size_t smem = (size_t)4 * (256 / head_size) * 2 * 16 * head_size * 2;       // 64 KB
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(group_attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(group_attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return fail("group_attention: cannot raise the shared memory limit");
        configured = true;
    }
#define LAUNCH_GROUP(D)                                                                                              \
    launch_kernel(g_dependent_launch != 0, group_attention_kernel<D>, grid, dim3(128), smem, s, (bf16*)out, ld_out,  \
                  (const bf16*)q, ld_q, (const bf16*)k_pages, (const bf16*)v_pages, block_table, max_blocks,         \
                  positions, token_item, n_heads, n_kv_heads, page_size, scale, window, chunk, max_chunks, part_acc, \
                  part_ml, counters)
    if (head_size == 64) LAUNCH_GROUP(64);
    else LAUNCH_GROUP(128);
#undef LAUNCH_GROUP
    return check_launch("group_attention_kernel");
}

// ---------------------------------------------------------------------------
// Layer norm, one warp per row, the row read once.  Each lane keeps up to HELD chunks of
// four values in registers (eight: rows up to 1024 wide; sixteen: up to 2048; measured at
// 2048 x 1600: 5.6 us with the row re-read for each pass); a wider row is re-read.
// Same arithmetic as the plain kernel: mean, variance of the centred values, then
// (x - mean) / sqrt(var + eps) * gain + shift, all in 32-bit; the output is bfloat16.
// ---------------------------------------------------------------------------
template <int HELD>
__global__ void __launch_bounds__(256)
layernorm_warp_kernel(bf16* __restrict__ out, const float* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, const int* __restrict__ rows, int n_rows, int width, float eps) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const float4* row = reinterpret_cast<const float4*>(x + (long)(rows ? rows[r] : r) * width);
    const int quads = width / 4;
    const bool held = quads <= 32 * HELD;
    float4 keep[HELD];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < HELD; i++) {
        keep[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (held && lane + 32 * i < quads) keep[i] = row[lane + 32 * i];
        sum += keep[i].x + keep[i].y + keep[i].z + keep[i].w;
    }
    if (!held)
        for (int q = lane; q < quads; q += 32) {
            const float4 v = row[q];
            sum += v.x + v.y + v.z + v.w;
        }
    const float mean = warp_sum(sum) / (float)width;
    float sq = 0.0f;
    if (held) {
#pragma unroll
        for (int i = 0; i < HELD; i++)
            if (lane + 32 * i < quads) {
                const float a = keep[i].x - mean, b = keep[i].y - mean, c = keep[i].z - mean, d = keep[i].w - mean;
                sq += a * a + b * b + c * c + d * d;
            }
    } else {
        for (int q = lane; q < quads; q += 32) {
            const float4 v = row[q];
            const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
            sq += a * a + b * b + c * c + d * d;
        }
    }
    const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    auto emit = [&](int q, const float4& v) {
        const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + q);
        const float4 b = __ldg(reinterpret_cast<const float4*>(beta) + q);
        __nv_bfloat162 lo = __floats2bfloat162_rn((v.x - mean) * inv * g.x + b.x, (v.y - mean) * inv * g.y + b.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn((v.z - mean) * inv * g.z + b.z, (v.w - mean) * inv * g.w + b.w);
        *reinterpret_cast<uint2*>(out + (long)r * width + q * 4) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    };
    if (held) {
#pragma unroll
        for (int i = 0; i < HELD; i++)
            if (lane + 32 * i < quads) emit(lane + 32 * i, keep[i]);
    } else {
        for (int q = lane; q < quads; q += 32) emit(q, row[q]);
    }
}

// x fp32 [*, width] (width a multiple of 4), out bfloat16 [n_rows, width]; rows: optional gather.
extern "C" int mllm_decode_layernorm(void* out, const float* x, const float* gamma, const float* beta, const int* rows,
                                     int n_rows, int width, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || width % 4 != 0) return fail("layernorm: the width must be a multiple of 4");
    if (width <= 1024)
        return launched(launch_kernel(g_dependent_launch != 0, layernorm_warp_kernel<8>, dim3((n_rows + 7) / 8), dim3(256), 0,
                                      (cudaStream_t)stream, (bf16*)out, x, gamma, beta, rows, n_rows, width, eps),
                        "layernorm_warp_kernel");
    return launched(launch_kernel(g_dependent_launch != 0, layernorm_warp_kernel<16>, dim3((n_rows + 7) / 8), dim3(256), 0,
                                  (cudaStream_t)stream, (bf16*)out, x, gamma, beta, rows, n_rows, width, eps),
                    "layernorm_warp_kernel");
}

// ---------------------------------------------------------------------------
// split_attention with built-in scratch, for callers that cannot allocate
// (see split_attention_static.h for who they are and what the limits mean).
// ---------------------------------------------------------------------------
#include "split_attention_static.h"

// Device memory.  In host code this name is only a handle for the symbol, not an address a
// kernel could use: the address is asked for once per device, below.
static __device__ __align__(256) unsigned char
    g_static_scratch[(MLLM_STATIC_ACC_FLOATS + MLLM_STATIC_ML_FLOATS) * sizeof(float) +
                     MLLM_STATIC_COUNTERS * sizeof(int)];

constexpr int STATIC_MAX_DEVICES = 64;
static unsigned char* g_static_address[STATIC_MAX_DEVICES] = {nullptr};

extern "C" int mllm_decode_split_attention_static(void* out, long ld_out, const void* q, long ld_q,
                                                  const void* k_pages, const void* v_pages, const int* block_table,
                                                  int max_blocks, const int* positions, const int* token_item,
                                                  int n_tokens, int n_heads, int n_kv_heads, int head_size,
                                                  int page_size, float scale, int window, int chunk, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_heads <= 0 || chunk <= 0 || page_size <= 0 || max_blocks <= 0 || head_size <= 0)
        return fail("split_attention_static: sizes must be positive");
    const long chunks = ((long)max_blocks * page_size + chunk - 1) / chunk;
    const long pairs = (long)n_tokens * n_heads;
    if (pairs > MLLM_STATIC_COUNTERS || pairs * chunks * 2 > MLLM_STATIC_ML_FLOATS ||
        pairs * chunks * head_size > MLLM_STATIC_ACC_FLOATS) {
        snprintf(g_error_text, MLLM_ERROR_BUFFER,
                 "split_attention_static: %d tokens x %d heads x %ld chunks x head size %d exceed the built-in scratch "
                 "(%d partial floats, %d max/sum floats, %d counters); use mllm_decode_split_attention with your own",
                 n_tokens, n_heads, chunks, head_size, MLLM_STATIC_ACC_FLOATS, MLLM_STATIC_ML_FLOATS,
                 MLLM_STATIC_COUNTERS);
        return 1;
    }
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= STATIC_MAX_DEVICES)
        return fail("split_attention_static: cannot tell the current device");
    if (g_static_address[device] == nullptr) {
        // set-up, once per device, with that device current
        void* address = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&address, g_static_scratch);
        if (e != cudaSuccess || address == nullptr) {
            snprintf(g_error_text, MLLM_ERROR_BUFFER, "split_attention_static: cudaGetSymbolAddress failed: %s",
                     cudaGetErrorString(e));
            return 2;
        }
        g_static_address[device] = static_cast<unsigned char*>(address);
    }
    float* part_acc = reinterpret_cast<float*>(g_static_address[device]);
    float* part_ml = part_acc + MLLM_STATIC_ACC_FLOATS;
    int* counters = reinterpret_cast<int*>(part_ml + MLLM_STATIC_ML_FLOATS);
    // The array keeps the last call's contents; the counters must start at zero.
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)pairs * sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) {
        snprintf(g_error_text, MLLM_ERROR_BUFFER, "split_attention_static: clearing the counters failed: %s",
                 cudaGetErrorString(e));
        return 2;
    }
    return mllm_decode_split_attention(out, ld_out, q, ld_q, k_pages, v_pages, block_table, max_blocks, positions,
                                       token_item, n_tokens, n_heads, n_kv_heads, head_size, page_size, scale, window,
                                       chunk, (int)chunks, part_acc, part_ml, counters, stream);
}
