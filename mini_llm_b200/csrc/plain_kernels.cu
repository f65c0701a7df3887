// Plain kernels: one straightforward SIMT kernel for every operation of a
// step.  With 32-bit element types they are the true 32-bit path of the whole
// model (scalar fp32 FMA, no tensor cores, no reduced-precision matrix mode);
// with bfloat16 element types they are the twin each fast kernel is checked
// against, and the kernel of last resort for sizes a fast kernel refuses.
// Sums, softmax and norm statistics are always 32-bit.
//
// Operations and their formulas follow the reference's CPU operators:
//   embedding   engine/src/embedding.c:9-15
//   layer norm  engine/src/layernorm.c:12-33
//   linear      engine/src/linear.c:5-19
//   attention   engine/src/attention.c:24-49 with the causal softmax of
//               engine/src/softmax.c:29-55, in the online form of
//               engine/src/attention.cu:98-123
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_plain)

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = table[id[t], :] (+ position_table[pos[t], :])
// ---------------------------------------------------------------------------
template <typename W>
__global__ void embed_kernel(float* __restrict__ out, const int* __restrict__ ids,
                             const int* __restrict__ positions, const W* __restrict__ table,
                             const W* __restrict__ position_table, int width) {
    dependents_may_start();
    wait_for_earlier_kernels();
    int t = blockIdx.x;
    long row = (long)ids[t] * width;
    if (position_table != nullptr) {
        long prow = (long)positions[t] * width;
        for (int d = threadIdx.x; d < width; d += blockDim.x)
            out[(long)t * width + d] = to_f32(table[row + d]) + to_f32(position_table[prow + d]);
    } else {
        for (int d = threadIdx.x; d < width; d += blockDim.x)
            out[(long)t * width + d] = to_f32(table[row + d]);
    }
}

// hidden[t, :] += position_table[pos[t], :]   (position encoding applied alone)
template <typename W>
__global__ void add_rows_kernel(float* __restrict__ hidden, const int* __restrict__ positions,
                                const W* __restrict__ table, int width) {
    int t = blockIdx.x;
    long prow = (long)positions[t] * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x)
        hidden[(long)t * width + d] += to_f32(table[prow + d]);
}

extern "C" int mllm_plain_embed(float* out, const int* ids, const int* positions, const void* table,
                                const void* position_table, int n_tokens, int width, int table_dtype,
                                void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = width >= 256 ? 256 : 64;
    if (table_dtype == DT_F32)
        launch_kernel(g_dependent_launch != 0, embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, out, ids, positions,
                      (const float*)table, (const float*)position_table, width);
    else if (table_dtype == DT_BF16)
        launch_kernel(g_dependent_launch != 0, embed_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, out, ids, positions,
                      (const bf16*)table, (const bf16*)position_table, width);
    else
        return fail("embed: unknown table dtype");
    return check_launch("embed_kernel");
}

extern "C" int mllm_plain_add_rows(float* hidden, const int* positions, const void* table, int n_tokens,
                                   int width, int table_dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = width >= 256 ? 256 : 64;
    if (table_dtype == DT_F32)
        add_rows_kernel<float><<<n_tokens, threads, 0, s>>>(hidden, positions, (const float*)table, width);
    else if (table_dtype == DT_BF16)
        add_rows_kernel<bf16><<<n_tokens, threads, 0, s>>>(hidden, positions, (const bf16*)table, width);
    else
        return fail("add_rows: unknown table dtype");
    return check_launch("add_rows_kernel");
}

// ---------------------------------------------------------------------------
// Layer norm, one block per row.  mean, then the variance of the centred
// values (biased), then (x - mean) * (1 / sqrt(var + eps)) * gamma + beta.
// `rows` (may be null) gathers: output row r is computed from input row
// rows[r].
// ---------------------------------------------------------------------------
template <typename O>
__global__ void layernorm_kernel(O* __restrict__ out, const float* __restrict__ x,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 const int* __restrict__ rows, int width, float eps) {
    __shared__ float scratch[33];
    int r = blockIdx.x;
    const float* row = x + (long)(rows ? rows[r] : r) * width;
    float sum = 0.0f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) sum += row[d];
    float mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.0f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float c = row[d] - mean;
        sq += c * c;
    }
    float var = block_sum(sq, scratch) / (float)width;
    float inv = 1.0f / sqrtf(var + eps);
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float n = (row[d] - mean) * inv;
        out[(long)r * width + d] = from_f32<O>(n * gamma[d] + beta[d]);
    }
}

extern "C" int mllm_plain_layernorm(void* out, const float* x, const float* gamma, const float* beta,
                                    const int* rows, int n_rows, int width, float eps, int out_dtype,
                                    void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
    if (out_dtype == DT_F32)
        layernorm_kernel<float><<<n_rows, threads, 0, s>>>((float*)out, x, gamma, beta, rows, width, eps);
    else if (out_dtype == DT_BF16)
        layernorm_kernel<bf16><<<n_rows, threads, 0, s>>>((bf16*)out, x, gamma, beta, rows, width, eps);
    else
        return fail("layernorm: unknown output dtype");
    return check_launch("layernorm_kernel");
}

// ---------------------------------------------------------------------------
// Linear: out[m, n] = epilogue(sum_k a[m, k] * w[n, k] + bias[n]).
// `w` is [N, K] with K contiguous.  64x64 tile, 256 threads, each 4x4
// outputs; the sum over k runs in order with fp32 FMA.
// ---------------------------------------------------------------------------
template <typename AT, typename WT, typename OT, int EPI>
__global__ void __launch_bounds__(256)
linear_plain_kernel(OT* __restrict__ out, const AT* __restrict__ a, const WT* __restrict__ w,
                    const float* __restrict__ bias, int M, int N, int K, long lda, long ldo) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            int r = i / BK, c = i % BK;
            int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f32(a[(long)gm * lda + gk]) : 0.0f;
            Ws[c][r] = (gn < N && gk < K) ? to_f32(w[(long)gn * K + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j] + (bias ? bias[gn] : 0.0f);
            long o = (long)gm * ldo + gn;
            if (EPI == EPI_ADD)
                out[o] = from_f32<OT>(to_f32(out[o]) + v);
            else
                out[o] = from_f32<OT>(apply_activation<EPI>(v));
        }
    }
}

template <typename AT, typename WT, typename OT>
static int launch_linear_plain(void* out, const void* a, const void* w, const float* bias, int M, int N, int K,
                               long lda, long ldo, int epilogue, cudaStream_t s) {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    OT* o = (OT*)out;
    const AT* ap = (const AT*)a;
    const WT* wp = (const WT*)w;
    switch (epilogue) {
    case EPI_STORE: linear_plain_kernel<AT, WT, OT, EPI_STORE><<<grid, 256, 0, s>>>(o, ap, wp, bias, M, N, K, lda, ldo); break;
    case EPI_GELU_TANH: linear_plain_kernel<AT, WT, OT, EPI_GELU_TANH><<<grid, 256, 0, s>>>(o, ap, wp, bias, M, N, K, lda, ldo); break;
    case EPI_GELU_ERF: linear_plain_kernel<AT, WT, OT, EPI_GELU_ERF><<<grid, 256, 0, s>>>(o, ap, wp, bias, M, N, K, lda, ldo); break;
    case EPI_ADD: linear_plain_kernel<AT, WT, OT, EPI_ADD><<<grid, 256, 0, s>>>(o, ap, wp, bias, M, N, K, lda, ldo); break;
    default: return fail("linear: unknown epilogue");
    }
    return check_launch("linear_plain_kernel");
}

// in_dtype: element type of `a` and `w`; out_dtype: element type of `out`
// (EPI_ADD needs a 32-bit `out`).  lda / ldo are row strides in elements.
extern "C" int mllm_plain_linear(void* out, const void* a, const void* w, const float* bias, int M, int N,
                                 int K, long lda, long ldo, int in_dtype, int out_dtype, int epilogue,
                                 void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return fail("linear: K must be positive");
    if ((M + 63) / 64 > 65535) return fail("linear: too many rows for one launch");
    if (epilogue == EPI_ADD && out_dtype != DT_F32) return fail("linear: the residual sum is kept in 32-bit");
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == DT_F32 && out_dtype == DT_F32)
        return launch_linear_plain<float, float, float>(out, a, w, bias, M, N, K, lda, ldo, epilogue, s);
    if (in_dtype == DT_BF16 && out_dtype == DT_BF16)
        return launch_linear_plain<bf16, bf16, bf16>(out, a, w, bias, M, N, K, lda, ldo, epilogue, s);
    if (in_dtype == DT_BF16 && out_dtype == DT_F32)
        return launch_linear_plain<bf16, bf16, float>(out, a, w, bias, M, N, K, lda, ldo, epilogue, s);
    return fail("linear: unsupported combination of element types");
}

// ---------------------------------------------------------------------------
// Store this step's keys and values into their pages.
// pages: [n_pages, page_size, width] per tensor, width = kv_heads * head_size.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void kv_store_kernel(T* __restrict__ k_pages, T* __restrict__ v_pages, const T* __restrict__ k_src,
                                const T* __restrict__ v_src, long ld_src, const int* __restrict__ positions,
                                const int* __restrict__ token_item, const int* __restrict__ block_table,
                                int max_blocks, int page_size, int width) {
    int t = blockIdx.x;
    int p = positions[t];
    int page = block_table[(long)token_item[t] * max_blocks + p / page_size];
    long dst = ((long)page * page_size + (p % page_size)) * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        k_pages[dst + d] = k_src[(long)t * ld_src + d];
        v_pages[dst + d] = v_src[(long)t * ld_src + d];
    }
}

extern "C" int mllm_plain_kv_store(void* k_pages, void* v_pages, const void* k_src, const void* v_src,
                                   long ld_src, const int* positions, const int* token_item,
                                   const int* block_table, int max_blocks, int page_size, int width,
                                   int n_tokens, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = width >= 256 ? 256 : 64;
    if (dtype == DT_F32)
        kv_store_kernel<float><<<n_tokens, threads, 0, s>>>((float*)k_pages, (float*)v_pages, (const float*)k_src,
                                                            (const float*)v_src, ld_src, positions, token_item,
                                                            block_table, max_blocks, page_size, width);
    else if (dtype == DT_BF16)
        kv_store_kernel<bf16><<<n_tokens, threads, 0, s>>>((bf16*)k_pages, (bf16*)v_pages, (const bf16*)k_src,
                                                           (const bf16*)v_src, ld_src, positions, token_item,
                                                           block_table, max_blocks, page_size, width);
    else
        return fail("kv_store: unknown dtype");
    return check_launch("kv_store_kernel");
}

// ---------------------------------------------------------------------------
// Causal attention over the paged cache, one block per (token, head).
// The query at absolute position p sees the keys at positions
// max(0, p - window + 1) .. p of its own request (window <= 0: all of them),
// read from the pages its block table names.  Four warps take the keys in
// turn, each with an online softmax; their states are merged at the end in a
// fixed order, so a token's result does not depend on the rest of the batch.
// ---------------------------------------------------------------------------
constexpr int ATT_PLAIN_MAX_HEAD = 256;

template <typename T>
__global__ void __launch_bounds__(128)
attention_plain_kernel(T* __restrict__ out, long ld_out, const T* __restrict__ q, long ld_q,
                       const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ positions,
                       const int* __restrict__ token_item, int n_heads, int n_kv_heads, int head_size,
                       int page_size, float scale, int window) {
    constexpr int R = ATT_PLAIN_MAX_HEAD / 32;
    int t = blockIdx.x, h = blockIdx.y;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int p = positions[t];
    const int* bt = block_table + (long)token_item[t] * max_blocks;
    int hk = h / (n_heads / n_kv_heads);
    int kv_width = n_kv_heads * head_size;

    float qr[R], acc[R];
#pragma unroll
    for (int i = 0; i < R; i++) {
        int d = lane + 32 * i;
        qr[i] = d < head_size ? to_f32(q[(long)t * ld_q + (long)h * head_size + d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    for (int j = lo + warp; j <= p; j += 4) {
        int page = bt[j / page_size];
        long base = ((long)page * page_size + (j % page_size)) * kv_width + (long)hk * head_size;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < R; i++) {
            int d = lane + 32 * i;
            if (d < head_size) s = fmaf(qr[i], to_f32(k_pages[base + d]), s);
        }
        s = warp_sum(s) * scale;
        float m_new = fmaxf(m, s);
        float c = expf(m - m_new);
        float e = expf(s - m_new);
        l = l * c + e;
#pragma unroll
        for (int i = 0; i < R; i++) {
            int d = lane + 32 * i;
            if (d < head_size) acc[i] = acc[i] * c + e * to_f32(v_pages[base + d]);
        }
        m = m_new;
    }

    __shared__ float sm_m[4], sm_l[4];
    __shared__ float sm_acc[4][ATT_PLAIN_MAX_HEAD];
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < R; i++) {
        int d = lane + 32 * i;
        if (d < head_size) sm_acc[warp][d] = acc[i];
    }
    __syncthreads();
    float big = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float total = 0.0f;
    float wgt[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        wgt[w] = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - big);
        total += sm_l[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < head_size; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) o += sm_acc[w][d] * wgt[w];
        out[(long)t * ld_out + (long)h * head_size + d] = from_f32<T>(o / total);
    }
}

extern "C" int mllm_plain_attention(void* out, long ld_out, const void* q, long ld_q, const void* k_pages,
                                    const void* v_pages, const int* block_table, int max_blocks,
                                    const int* positions, const int* token_item, int n_tokens, int n_heads,
                                    int n_kv_heads, int head_size, int page_size, float scale, int window,
                                    int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (head_size <= 0 || head_size > ATT_PLAIN_MAX_HEAD) return fail("attention: head size must be in 1..256");
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        return fail("attention: the number of heads must be a multiple of the number of key/value heads");
    if (n_heads > 65535) return fail("attention: too many heads for one launch");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, n_heads);
    if (dtype == DT_F32)
        attention_plain_kernel<float><<<grid, 128, 0, s>>>((float*)out, ld_out, (const float*)q, ld_q,
                                                           (const float*)k_pages, (const float*)v_pages, block_table,
                                                           max_blocks, positions, token_item, n_heads, n_kv_heads,
                                                           head_size, page_size, scale, window);
    else if (dtype == DT_BF16)
        attention_plain_kernel<bf16><<<grid, 128, 0, s>>>((bf16*)out, ld_out, (const bf16*)q, ld_q,
                                                          (const bf16*)k_pages, (const bf16*)v_pages, block_table,
                                                          max_blocks, positions, token_item, n_heads, n_kv_heads,
                                                          head_size, page_size, scale, window);
    else
        return fail("attention: unknown dtype");
    return check_launch("attention_plain_kernel");
}

// The current device, for a benchmark's record: name, compute capability, SM count, memory,
// runtime and driver versions (the reference's gpt2_gpu_device_info, engine/src/gpt2_gpu.cu:369-383).
// values: [major, minor, SMs, runtime version, driver version]; memory in bytes.
extern "C" int mllm_plain_device_info(char* name, int name_bytes, int* values, long* memory_bytes) {
    int device = 0;
    cudaDeviceProp properties;
    if (cudaGetDevice(&device) != cudaSuccess || cudaGetDeviceProperties(&properties, device) != cudaSuccess)
        return fail("device_info: no CUDA device");
    snprintf(name, (size_t)name_bytes, "%s", properties.name);
    values[0] = properties.major;
    values[1] = properties.minor;
    values[2] = properties.multiProcessorCount;
    *memory_bytes = (long)properties.totalGlobalMem;
    if (cudaRuntimeGetVersion(&values[3]) != cudaSuccess || cudaDriverGetVersion(&values[4]) != cudaSuccess)
        return fail("device_info: cannot read the versions");
    return 0;
}
