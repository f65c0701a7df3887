// Sampling on the device: greedy, temperature and nucleus (top-p), one block
// per row of logits.
//
// Greedy follows the reference's argmax rules (engine/include/argmax.h:10-13,
// engine/src/argmax.cu:8-18): the first index wins a tie, a NaN beats every
// number and the first NaN wins.  The reference's engine samples greedily
// only; its command line (scripts/complete.py:116-123) adds temperature and
// top-p, with temperature <= 0 meaning greedy.  Here those are done by the
// Gumbel-max rule: the chosen token is argmax_v(logit_v / T + g_v) over the
// kept tokens, g_v = -log(-log(u_v)), u_v a hash of (seed, counter, v).  The
// draw depends on nothing but the row's own logits and its (seed, counter),
// so it is the same in every batch, and a host twin can repeat it.
#include "common.cuh"

MLLM_DEFINE_ERROR_API(mllm_sampling)

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Uniform in (0, 1) with 24 bits, from (seed, counter, index).
__device__ __forceinline__ float uniform_of(uint64_t seed, uint32_t counter, uint32_t index) {
    uint64_t h = mix64(mix64(seed ^ ((uint64_t)counter << 32)) ^ (uint64_t)index);
    return ((float)(uint32_t)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ bool better(float va, int ia, float vb, int ib) {
    bool na = va != va, nb = vb != vb;
    if (ia < 0) return false;
    if (ib < 0) return true;
    if (na != nb) return na;
    if (na) return ia < ib;
    if (va != vb) return va > vb;
    return ia < ib;
}

__device__ __forceinline__ void block_argmax(float& v, int& i, float* sv, int* si) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    if (warp == 0) {
        v = lane < n_warps ? sv[lane] : 0.0f;
        i = lane < n_warps ? si[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, v, o);
            int oi = __shfl_xor_sync(0xffffffffu, i, o);
            if (better(ov, oi, v, i)) { v = ov; i = oi; }
        }
        if (lane == 0) { sv[0] = v; si[0] = i; }
    }
    __syncthreads();
    v = sv[0];
    i = si[0];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// temperature[r] <= 0: greedy.  top_p[r] >= 1: no nucleus cut.
// The nucleus is the smallest set of most probable tokens whose probability
// reaches top_p, ties at its edge included: tokens with p >= t*, where t* is
// the largest t with sum_{p_v >= t} p_v >= top_p, found by bisection on the
// bit pattern of t.
// With `cached` the row's probabilities are computed once into dynamic shared memory (vocab
// floats) and the bisection's thirty passes read them there: the same values, compared and
// summed in the same order as without, so the draw is bit for bit the same; it only stops
// costing thirty passes of exponentials over global memory.
__global__ void __launch_bounds__(1024)
sample_rows_kernel(int* __restrict__ out, const float* __restrict__ logits, long ld, int vocab,
                   const float* __restrict__ temperature, const float* __restrict__ top_p,
                   const unsigned long long* __restrict__ seeds, const int* __restrict__ counters,
                   int only_nucleus, int cached) {
    extern __shared__ float probs[];
    __shared__ float sv[33];
    __shared__ int si[32];
    dependents_may_start();
    wait_for_earlier_kernels();
    int r = blockIdx.x;
    const float* x = logits + (long)r * ld;
    float temp = temperature ? temperature[r] : 0.0f;
    // only_nucleus: the sliced kernel has drawn every row but those with a nucleus cut
    if (only_nucleus && !(temp > 0.0f && top_p != nullptr && top_p[r] < 1.0f)) return;
    float best = 0.0f;
    int best_i = -1;

    if (!(temp > 0.0f)) {
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
            float xv = x[v];
            if (better(xv, v, best, best_i)) { best = xv; best_i = v; }
        }
        block_argmax(best, best_i, sv, si);
        if (threadIdx.x == 0) out[r] = best_i;
        return;
    }

    float inv_t = 1.0f / temp;
    float nucleus = top_p ? top_p[r] : 1.0f;
    float cut = 0.0f;       // keep tokens with probability >= cut
    float big = 0.0f, z = 1.0f;
    if (nucleus < 1.0f) {
        float mx = -INFINITY;
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) mx = fmaxf(mx, x[v]);
        big = block_max(mx, sv);
        float sum = 0.0f;
        for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
            const float e = expf((x[v] - big) * inv_t);
            if (cached) probs[v] = e;
            sum += e;
        }
        z = block_sum(sum, sv);
        if (cached)
            for (int v = threadIdx.x; v < vocab; v += blockDim.x) probs[v] = probs[v] / z;      // each thread its own entries
        unsigned lo = 0u, hi = 0x3f800000u;      // bit patterns of 0.0f and 1.0f
        while (lo < hi) {
            unsigned mid = lo + (hi - lo + 1u) / 2u;
            float t = __uint_as_float(mid);
            float mass = 0.0f;
            if (cached) {
                for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
                    const float pv = probs[v];
                    if (pv >= t) mass += pv;
                }
            } else {
                for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
                    float pv = expf((x[v] - big) * inv_t) / z;
                    if (pv >= t) mass += pv;
                }
            }
            mass = block_sum(mass, sv);
            if (mass >= nucleus) lo = mid; else hi = mid - 1u;
        }
        cut = __uint_as_float(lo);
    }

    unsigned long long seed = seeds ? seeds[r] : 0ull;
    unsigned counter = counters ? (unsigned)counters[r] : 0u;
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
        float xv = x[v];
        if (nucleus < 1.0f && !((cached ? probs[v] : expf((xv - big) * inv_t) / z) >= cut)) continue;
        float u = uniform_of(seed, counter, (unsigned)v);
        float score = xv * inv_t - logf(-logf(u));
        if (better(score, v, best, best_i)) { best = score; best_i = v; }
    }
    block_argmax(best, best_i, sv, si);
    if (threadIdx.x == 0) out[r] = best_i;
}

// The same draw for rows without a nucleus cut, spread over SLICES blocks per row: each
// block finds the best candidate of its slice of the vocabulary, and the block that
// finishes last for a row picks the best of the slices (ties to the lower index, so the
// result is the one-block kernel's).  Rows with top_p < 1 are left to sample_rows_kernel.
// scratch: floats [rows * SLICES], ints [rows * SLICES], zeroed int counters [rows].
constexpr int SAMPLE_SLICES = 32;

__global__ void __launch_bounds__(256)
sample_rows_sliced_kernel(int* __restrict__ out, const float* __restrict__ logits, long ld, int vocab,
                          const float* __restrict__ temperature, const float* __restrict__ top_p,
                          const unsigned long long* __restrict__ seeds, const int* __restrict__ counters,
                          float* __restrict__ part_value, int* __restrict__ part_index, int* __restrict__ done) {
    __shared__ float sv[33];
    __shared__ int si[32];
    __shared__ int is_last;
    dependents_may_start();
    wait_for_earlier_kernels();
    const int r = blockIdx.x, slice = blockIdx.y;
    if (top_p != nullptr && top_p[r] < 1.0f && temperature != nullptr && temperature[r] > 0.0f) return;
    const float* x = logits + (long)r * ld;
    const float temp = temperature ? temperature[r] : 0.0f;
    const int per = (vocab + SAMPLE_SLICES - 1) / SAMPLE_SLICES;
    const int begin = slice * per, end = min(vocab, begin + per);
    float best = 0.0f;
    int best_i = -1;
    if (!(temp > 0.0f)) {
        for (int v = begin + threadIdx.x; v < end; v += blockDim.x) {
            float xv = x[v];
            if (better(xv, v, best, best_i)) { best = xv; best_i = v; }
        }
    } else {
        const float inv_t = 1.0f / temp;
        const unsigned long long seed = seeds ? seeds[r] : 0ull;
        const unsigned counter = counters ? (unsigned)counters[r] : 0u;
        for (int v = begin + threadIdx.x; v < end; v += blockDim.x) {
            float score = x[v] * inv_t - logf(-logf(uniform_of(seed, counter, (unsigned)v)));
            if (better(score, v, best, best_i)) { best = score; best_i = v; }
        }
    }
    block_argmax(best, best_i, sv, si);
    if (threadIdx.x == 0) {
        part_value[r * SAMPLE_SLICES + slice] = best;
        part_index[r * SAMPLE_SLICES + slice] = best_i;
        __threadfence();
        int ticket = atomicAdd(&done[r], 1);
        is_last = ticket == SAMPLE_SLICES - 1;
        if (is_last) done[r] = 0;
    }
    __syncthreads();
    if (!is_last || threadIdx.x >= 32) return;
    __threadfence();
    float v = __ldcg(part_value + r * SAMPLE_SLICES + threadIdx.x);
    int i = __ldcg(part_index + r * SAMPLE_SLICES + threadIdx.x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    if (threadIdx.x == 0) out[r] = i;
}

// ---------------------------------------------------------------------------
// Rows with a nucleus cut, four CTAs (a cluster) per row.  Each thread keeps its share of the
// row's probabilities in registers (PER of them: the row's entries 4096 i + 1024 rank +
// thread), so a pass of the bisection is PER compares and adds, a sum over the block, and an
// exchange of the four blocks' sums through distributed shared memory, added in rank order:
// the thirty passes cost microseconds instead of thirty sweeps over shared memory, and the
// result depends on nothing but the row.  Takes vocabularies of up to 4096 PER entries.
// ---------------------------------------------------------------------------
constexpr int NUCLEUS_CLUSTER = 4;

__device__ __forceinline__ uint32_t cluster_rank_of_cta() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float read_float_of_rank(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ int read_int_of_rank(const int* local, uint32_t rank) {
    uint32_t remote;
    int v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
}

// The blocks' values, each already the same in all threads of its block, combined over the
// cluster in rank order.  `slots`: two floats of shared memory, used in turn (`turn` counts
// the exchanges), so that one cluster barrier per exchange is enough.
template <bool MAX>
__device__ __forceinline__ float cluster_combine(float v, float* slots, int& turn) {
    float* mine = slots + (turn & 1);
    turn++;
    if (threadIdx.x == 0) *mine = v;
    cluster_sync_all();
    float total = MAX ? -INFINITY : 0.0f;
#pragma unroll
    for (uint32_t rank = 0; rank < NUCLEUS_CLUSTER; rank++) {
        const float other = read_float_of_rank(mine, rank);
        total = MAX ? fmaxf(total, other) : total + other;
    }
    return total;
}

template <int PER>
__global__ void __cluster_dims__(NUCLEUS_CLUSTER, 1, 1) __launch_bounds__(1024)
nucleus_rows_kernel(int* __restrict__ out, const float* __restrict__ logits, long ld, int vocab,
                    const float* __restrict__ temperature, const float* __restrict__ top_p,
                    const unsigned long long* __restrict__ seeds, const int* __restrict__ counters) {
    __shared__ float sv[33];
    __shared__ int si[32];
    __shared__ float slots[2];
    __shared__ float best_value;
    __shared__ int best_index;
    dependents_may_start();
    wait_for_earlier_kernels();
    const int r = blockIdx.x / NUCLEUS_CLUSTER;
    const uint32_t rank = cluster_rank_of_cta();
    const float temp = temperature[r], nucleus = top_p[r];
    if (!(temp > 0.0f && nucleus < 1.0f)) return;          // the whole cluster alike: drawn by the sliced kernel
    const float* x = logits + (long)r * ld;
    const float inv_t = 1.0f / temp;
    const int first = (int)rank * 1024 + threadIdx.x;
    int turn = 0;
    float p[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int v = first + i * (NUCLEUS_CLUSTER * 1024);
        p[i] = v < vocab ? x[v] : -INFINITY;
        mx = fmaxf(mx, p[i]);
    }
    const float big = cluster_combine<true>(block_max(mx, sv), slots, turn);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        p[i] = expf((p[i] - big) * inv_t);                  // 0 for the entries past the vocabulary
        sum += p[i];
    }
    const float z = cluster_combine<false>(block_sum(sum, sv), slots, turn);
#pragma unroll
    for (int i = 0; i < PER; i++) p[i] = p[i] / z;
    // the largest t with sum over p >= t of p >= nucleus, by bisection on t's bit pattern
    unsigned lo = 0u, hi = 0x3f800000u;
    while (lo < hi) {
        const unsigned mid = lo + (hi - lo + 1u) / 2u;
        const float t = __uint_as_float(mid);
        float mass = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; i++)
            if (p[i] >= t) mass += p[i];
        mass = cluster_combine<false>(block_sum(mass, sv), slots, turn);
        if (mass >= nucleus) lo = mid; else hi = mid - 1u;
    }
    const float cut = __uint_as_float(lo);
    const unsigned long long seed = seeds ? seeds[r] : 0ull;
    const unsigned counter = counters ? (unsigned)counters[r] : 0u;
    float best = 0.0f;
    int best_i = -1;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int v = first + i * (NUCLEUS_CLUSTER * 1024);
        if (v >= vocab || !(p[i] >= cut)) continue;
        const float score = x[v] * inv_t - logf(-logf(uniform_of(seed, counter, (unsigned)v)));
        if (better(score, v, best, best_i)) { best = score; best_i = v; }
    }
    block_argmax(best, best_i, sv, si);
    if (threadIdx.x == 0) {
        best_value = best;
        best_index = best_i;
    }
    cluster_sync_all();
    if (rank == 0 && threadIdx.x == 0) {
        for (uint32_t other = 1; other < NUCLEUS_CLUSTER; other++) {
            const float ov = read_float_of_rank(&best_value, other);
            const int oi = read_int_of_rank(&best_index, other);
            if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
        }
        out[r] = best_i;
    }
    cluster_sync_all();                                     // nobody leaves while its shared memory may be read
}

constexpr int NUCLEUS_PER = 16;       // vocabularies of up to 65,536 entries

// Launches the one-block-per-row kernel, with the row's probabilities kept in shared memory
// when the vocabulary fits there.
static int launch_sample_rows(int* out, const float* logits, long ld, int n_rows, int vocab, const float* temperature,
                              const float* top_p, const unsigned long long* seeds, const int* counters, int only_nucleus,
                              cudaStream_t s) {
    static int smem_limit = -1;
    if (smem_limit < 0) {
        int device = 0, optin = 0;
        cudaFuncAttributes attributes;
        if (cudaGetDevice(&device) == cudaSuccess &&
            cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) == cudaSuccess &&
            cudaFuncGetAttributes(&attributes, sample_rows_kernel) == cudaSuccess) {
            const int room = optin - (int)attributes.sharedSizeBytes - 1024;
            smem_limit = (room > 0 && cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                           room) == cudaSuccess) ? room : 0;
        } else {
            smem_limit = 0;
        }
        cudaGetLastError();
    }
    const bool cached = top_p != nullptr && (long)vocab * 4 <= (long)smem_limit;
    return launched(launch_kernel(g_dependent_launch != 0, sample_rows_kernel, dim3(n_rows), dim3(1024),
                                  cached ? (size_t)vocab * 4 : 0, s, out, logits, ld, vocab, temperature, top_p, seeds, counters,
                                  only_nucleus, cached ? 1 : 0),
                    "sample_rows_kernel");
}

// The rows with a nucleus cut only: by the cluster kernel when the vocabulary fits its
// registers, else by the one-block kernel.
static int launch_nucleus_rows(int* out, const float* logits, long ld, int n_rows, int vocab, const float* temperature,
                               const float* top_p, const unsigned long long* seeds, const int* counters, cudaStream_t s) {
    if (temperature == nullptr || top_p == nullptr) return 0;        // no row has a cut
    if (vocab <= NUCLEUS_CLUSTER * 1024 * NUCLEUS_PER) {
        // (the cluster's size is part of the kernel's declaration)
        return launched(launch_kernel(g_dependent_launch != 0, nucleus_rows_kernel<NUCLEUS_PER>, dim3(n_rows * NUCLEUS_CLUSTER),
                                      dim3(1024), 0, s, out, logits, ld, vocab, temperature, top_p, seeds, counters),
                        "nucleus_rows_kernel");
    }
    return launch_sample_rows(out, logits, ld, n_rows, vocab, temperature, top_p, seeds, counters, 1, s);
}

// any_nucleus: some row has temperature > 0 and top_p < 1 (the host knows); those rows are
// then drawn by the one-block kernel, which skips all others.
extern "C" int mllm_sampling_sample_rows_sliced(int* out, const float* logits, long ld, int n_rows, int vocab,
                                                const float* temperature, const float* top_p,
                                                const unsigned long long* seeds, const int* counters,
                                                float* part_value, int* part_index, int* done, int any_nucleus,
                                                void* stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return fail("sample_rows: empty vocabulary");
    cudaStream_t s = (cudaStream_t)stream;
    int rc = launched(launch_kernel(g_dependent_launch != 0, sample_rows_sliced_kernel, dim3(n_rows, SAMPLE_SLICES), dim3(256), 0, s,
                                    out, logits, ld, vocab, temperature, top_p, seeds, counters, part_value, part_index, done),
                      "sample_rows_sliced_kernel");
    if (rc == 0 && any_nucleus) rc = launch_nucleus_rows(out, logits, ld, n_rows, vocab, temperature, top_p, seeds, counters, s);
    return rc;
}

// Only the rows with a nucleus cut (temperature > 0 and top_p < 1); every other row of
// `out` is left as it is.
extern "C" int mllm_sampling_sample_rows_nucleus(int* out, const float* logits, long ld, int n_rows, int vocab,
                                                 const float* temperature, const float* top_p,
                                                 const unsigned long long* seeds, const int* counters, void* stream) {
    if (n_rows <= 0) return 0;
    return launch_nucleus_rows(out, logits, ld, n_rows, vocab, temperature, top_p, seeds, counters, (cudaStream_t)stream);
}

extern "C" int mllm_sampling_sample_rows(int* out, const float* logits, long ld, int n_rows, int vocab,
                                         const float* temperature, const float* top_p,
                                         const unsigned long long* seeds, const int* counters, void* stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return fail("sample_rows: empty vocabulary");
    return launch_sample_rows(out, logits, ld, n_rows, vocab, temperature, top_p, seeds, counters, 0, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Feeding a request its own last sampled token without a trip to the host.
//   keep_tokens     kept[slots[r]] = tokens[r] for every sampled row r whose slots[r] >= 0
//   resolve_tokens  ids[t] = kept[-1 - ids[t]] for every id below zero
// `kept` has one entry per request slot.  The reference keeps the sampled token of its
// single-sequence greedy loop on the device in the same spirit
// (engine/src/gpt2_gpu_greedy.cu:80-119).
// ---------------------------------------------------------------------------
__global__ void keep_tokens_kernel(int* __restrict__ kept, const int* __restrict__ slots,
                                   const int* __restrict__ tokens, int n, int n_kept) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    const int slot = slots[r];
    if (slot >= 0 && slot < n_kept) kept[slot] = tokens[r];
}

__global__ void resolve_tokens_kernel(int* __restrict__ ids, const int* __restrict__ kept, int n, int n_kept) {
    dependents_may_start();
    wait_for_earlier_kernels();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const int id = ids[t];
    if (id >= 0) return;
    const int slot = -1 - id;
    ids[t] = slot < n_kept ? kept[slot] : 0;
}

extern "C" int mllm_sampling_keep_tokens(int* kept, const int* slots, const int* tokens, int n, int n_kept,
                                         void* stream) {
    if (n <= 0) return 0;
    return launched(launch_kernel(g_dependent_launch != 0, keep_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0,
                                  (cudaStream_t)stream, kept, slots, tokens, n, n_kept),
                    "keep_tokens_kernel");
}

extern "C" int mllm_sampling_resolve_tokens(int* ids, const int* kept, int n, int n_kept, void* stream) {
    if (n <= 0) return 0;
    return launched(launch_kernel(g_dependent_launch != 0, resolve_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0,
                                  (cudaStream_t)stream, ids, kept, n, n_kept),
                    "resolve_tokens_kernel");
}
