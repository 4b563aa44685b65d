// A mixture-of-experts router with independent (sigmoid) scores, and the sum that ends such a layer.
//
// moe_route_topk: from every token's router logits z [experts] (float32), the `top` experts with
// the largest logits (the sigmoid keeps the order; of equal logits the lower index wins) and for
// each pair p = m * top + j its score s = sigmoid(z) and s^2.  It counts the pairs of every expert
// and writes them out grouped by expert, as the grouped products read them: perm[i] is the pair at
// place i, off[e] .. off[e + 1] the places of expert e.  One block.
//
// moe_route_softmax: the same output for a router with softmax scores s = softmax(z) over all experts.  Experts are
// CHOSEN by s + correction (a float32 value per expert, or none), only among the experts of the `keep` best of
// `n_groups` equal runs of neighbouring experts (a run's score is its largest choice score; n_groups <= 1: all
// experts), ties to the lower index; a pair's WEIGHT is its s divided by the sum of the token's chosen s (+ 1e-20),
// times `scale`.  Scores that are not allowed do not count as 0: choice scores may be negative.
//
// The experts of moe_route_topk act on the scaled input, expert(s x) = Wdown relu(Wup (s x))^2, which for s > 0
// is s^2 Wdown relu(Wup x)^2: the products run on x itself and
// moe_combine_gated: out[m] = sum_j s_p^2 z[place of pair p] + sigmoid(g_m) * shared[m]
// applies the squares at the end, with a shared expert's output behind a gate of its own logit
// (both optional).
#include "common.cuh"

namespace {

constexpr int RT_THREADS = 1024, MAX_TOP = 16;

__global__ void moe_route_topk_kernel(const float* __restrict__ z, long long ldz, int n_experts, int top, int M,
                                      int* __restrict__ perm, int* __restrict__ off, int* __restrict__ pair_expert,
                                      float* __restrict__ pair_score, float* __restrict__ pair_score2) {
    ti_pdl_trigger();
    extern __shared__ int cnt[];         // [n_experts] counts, then [n_experts + 1] offsets, then [n_experts] cursors
    int* offs = cnt + n_experts;
    int* cur = offs + n_experts + 1;
    ti_pdl_sync();
    z = ti_dependent(z);
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        const float* zr = z + (size_t)m * ldz;
        int chosen[MAX_TOP];
        for (int j = 0; j < top; j++) {
            int best = -1;
            float bz = 0.f;
            for (int e = 0; e < n_experts; e++) {
                bool taken = false;
                for (int i = 0; i < j; i++) taken |= chosen[i] == e;
                if (taken) continue;
                const float x = zr[e];
                if (best < 0 || x > bz) { best = e; bz = x; }      // a row of NaN keeps the lowest free index
            }
            chosen[j] = best;
            const int p = m * top + j;
            const float s = 1.0f / (1.0f + expf(-bz));
            pair_expert[p] = best;
            pair_score[p] = s;
            pair_score2[p] = s * s;
            atomicAdd(&cnt[best], 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0;
        for (int e = 0; e < n_experts; e++) { offs[e] = a; a += cnt[e]; }
        offs[n_experts] = a;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) off[e] = offs[e];
    const int P = M * top;
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = pair_expert[p];
        perm[offs[e] + atomicAdd(&cur[e], 1)] = p;
    }
}

// what both routers end with: the pairs of every expert counted in cnt[], written out grouped by expert
__device__ __forceinline__ void group_pairs(int* cnt, int* offs, int* cur, int n_experts, int P, const int* pair_expert,
                                            int* __restrict__ perm, int* __restrict__ off) {
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0;
        for (int e = 0; e < n_experts; e++) { offs[e] = a; a += cnt[e]; }
        offs[n_experts] = a;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) off[e] = offs[e];
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = pair_expert[p];
        perm[offs[e] + atomicAdd(&cur[e], 1)] = p;
    }
}

constexpr int MAX_GROUPS = 64;

__global__ void moe_route_softmax_kernel(const float* __restrict__ z, long long ldz, const float* __restrict__ correction,
                                         int n_experts, int top, int n_groups, int keep, float scale, int M,
                                         int* __restrict__ perm, int* __restrict__ off, int* __restrict__ pair_expert,
                                         float* __restrict__ pair_w) {
    ti_pdl_trigger();
    extern __shared__ int cnt[];         // [n_experts] counts, then [n_experts + 1] offsets, then [n_experts] cursors
    int* offs = cnt + n_experts;
    int* cur = offs + n_experts + 1;
    ti_pdl_sync();
    z = ti_dependent(z);
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    const int per = n_groups > 1 ? n_experts / n_groups : n_experts;
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        const float* zr = z + (size_t)m * ldz;
        float zmax = -INFINITY;
        for (int e = 0; e < n_experts; e++) zmax = fmaxf(zmax, zr[e]);
        float sum = 0.f;
        for (int e = 0; e < n_experts; e++) sum += expf(zr[e] - zmax);
        const float inv = 1.0f / sum;
        auto score = [&](int e) { return expf(zr[e] - zmax) * inv; };
        auto choice = [&](int e) { return score(e) + (correction ? correction[e] : 0.f); };
        unsigned long long open = ~0ull;                 // bit g: experts of run g may be chosen
        if (n_groups > 1 && keep < n_groups) {
            open = 0ull;
            for (int j = 0; j < keep; j++) {
                int best = -1;
                float bs = 0.f;
                for (int g = 0; g < n_groups; g++) {
                    if (open >> g & 1ull) continue;
                    float gs = -INFINITY;
                    for (int e = g * per; e < (g + 1) * per; e++) gs = fmaxf(gs, choice(e));
                    if (best < 0 || gs > bs) { best = g; bs = gs; }
                }
                open |= 1ull << best;
            }
        }
        int chosen[MAX_TOP];
        float s_of[MAX_TOP];
        float total = 0.f;
        for (int j = 0; j < top; j++) {
            int best = -1;
            float bc = 0.f;
            for (int e = 0; e < n_experts; e++) {
                if (n_groups > 1 && !(open >> (e / per) & 1ull)) continue;
                bool taken = false;
                for (int i = 0; i < j; i++) taken |= chosen[i] == e;
                if (taken) continue;
                const float c = choice(e);
                if (best < 0 || c > bc) { best = e; bc = c; }      // a row of NaN keeps the lowest free index
            }
            chosen[j] = best;
            s_of[j] = score(best);
            total += s_of[j];
        }
        const float norm = scale / (total + 1e-20f);
        for (int j = 0; j < top; j++) {
            const int p = m * top + j;
            pair_expert[p] = chosen[j];
            pair_w[p] = s_of[j] * norm;
            atomicAdd(&cnt[chosen[j]], 1);
        }
    }
    group_pairs(cnt, offs, cur, n_experts, M * top, pair_expert, perm, off);
}

template <typename T>
__global__ void moe_combine_gated_kernel(const T* __restrict__ z, const int* __restrict__ place_of_pair,
                                         const float* __restrict__ pair_w, const T* __restrict__ shared_out,
                                         const float* __restrict__ gate_logit, long long gate_stride, T* __restrict__ out, int H,
                                         int top) {
    ti_pdl_trigger();
    ti_pdl_sync();
    z = ti_dependent(z); place_of_pair = ti_dependent(place_of_pair); pair_w = ti_dependent(pair_w);
    shared_out = ti_dependent(shared_out); gate_logit = ti_dependent(gate_logit);
    const size_t m = blockIdx.x;
    const float g = (shared_out && gate_logit) ? 1.0f / (1.0f + expf(-gate_logit[m * gate_stride])) : 1.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; j++) {
            const size_t p = m * top + j;
            const size_t at = place_of_pair ? (size_t)place_of_pair[p] : p;
            s = fmaf(pair_w ? pair_w[p] : 1.f, to_f32(z[at * H + i]), s);
        }
        if (shared_out) s = fmaf(g, to_f32(shared_out[m * H + i]), s);
        out[m * H + i] = from_f32<T>(s);
    }
}

}  // namespace

// z: float32 [M, >= n_experts] with row stride ldz; perm: int32 [M * top]; off: int32 [n_experts + 1]; pair_expert: int32
// scratch [M * top]; pair_score, pair_score2: float32 [M * top].
extern "C" int ti_moe_route_topk(const float* z, long long ldz, int n_experts, int top, int M, int* perm, int* off,
                                 int* pair_expert, float* pair_score, float* pair_score2, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_experts > 0 && top >= 1 && top <= n_experts && top <= MAX_TOP && ldz >= n_experts,
               "moe_route_topk: bad sizes (%d experts, %d per token; at most %d per token)", n_experts, top, MAX_TOP);
    const size_t smem = (size_t)(3 * n_experts + 1) * sizeof(int);
    TI_REQUIRE(smem <= 48 * 1024, "moe_route_topk: %d experts are too many", n_experts);
    TI_CUDA(ti_launch_class<1>(moe_route_topk_kernel, dim3(1), dim3(RT_THREADS), smem, stream, z, ldz, n_experts, top, M, perm, off,
                               pair_expert, pair_score, pair_score2));
    TI_CHECK_LAUNCH("moe_route_topk");
    return 0;
}

// z: float32 [M, >= n_experts] with row stride ldz; correction: float32 [n_experts] or null; n_groups <= 1: no runs; perm: int32
// [M * top]; off: int32 [n_experts + 1]; pair_expert: int32 scratch [M * top]; pair_w: float32 [M * top].
extern "C" int ti_moe_route_softmax(const float* z, long long ldz, const float* correction, int n_experts, int top, int n_groups,
                                    int keep, float scale, int M, int* perm, int* off, int* pair_expert, float* pair_w,
                                    cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_experts > 0 && top >= 1 && top <= n_experts && top <= MAX_TOP && ldz >= n_experts,
               "moe_route_softmax: bad sizes (%d experts, %d per token; at most %d per token)", n_experts, top, MAX_TOP);
    if (n_groups > 1)
        TI_REQUIRE(n_groups <= MAX_GROUPS && n_experts % n_groups == 0 && keep >= 1 && keep <= n_groups &&
                   (long long)keep * (n_experts / n_groups) >= top,
                   "moe_route_softmax: %d experts in %d runs of which %d stay, %d per token (at most %d runs)", n_experts, n_groups, keep,
                   top, MAX_GROUPS);
    const size_t smem = (size_t)(3 * n_experts + 1) * sizeof(int);
    TI_REQUIRE(smem <= 48 * 1024, "moe_route_softmax: %d experts are too many", n_experts);
    TI_CUDA(ti_launch_class<1>(moe_route_softmax_kernel, dim3(1), dim3(RT_THREADS), smem, stream, z, ldz, correction, n_experts, top,
                               n_groups, keep, scale, M, perm, off, pair_expert, pair_w));
    TI_CHECK_LAUNCH("moe_route_softmax");
    return 0;
}

// z: [places, H] of the engine's type; place_of_pair: int32 [M * top] or null (pair p sits at row p); pair_w: float32
// [M * top] or null (ones); shared_out: [M, H] or null; gate_logit: float32, token m's at gate_logit[m * gate_stride], or null.
extern "C" int ti_moe_combine_gated(const void* z, const int* place_of_pair, const float* pair_w, const void* shared_out,
                                    const float* gate_logit, long long gate_stride, void* out, int M, int H, int top, int dtype,
                                    cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && H > 0 && top > 0, "moe_combine_gated: bad sizes");
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(moe_combine_gated_kernel<T>, dim3(M), dim3(H <= 256 ? 64 : 256), 0, stream, (const T*)z, place_of_pair,
                                   pair_w, (const T*)shared_out, gate_logit, gate_stride, (T*)out, H, top));
        TI_CHECK_LAUNCH("moe_combine_gated");
        return 0;
    });
}
