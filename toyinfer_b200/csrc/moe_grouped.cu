// Mixture-of-experts feed-forward: tokens grouped by expert, one product kernel over all groups.
//
// A step has P = tokens * top (token, choice) pairs; pair p = m * top + j uses expert
// e_p.  `moe_route_table` takes e_p from a table indexed by the token's id (a router
// without arithmetic: table[id, j]), counts the pairs of every expert and writes them out
// grouped by expert: perm[i] is the pair at place i, off[e] .. off[e + 1] the places of expert e.
// The order inside a group is whatever the atomics gave; no result depends on it, since every
// pair's rows are computed for themselves.
//
// `moe_grouped` is the product kernel, used twice:
//   first product   rows of x gathered by pair (token perm[i] / top), expert e's gate and up
//                   matrices, then the expert's activation, into y[i] (places, grouped)
//   second product  rows y[i], expert e's down matrix, result scattered to z[perm[i]] (pairs in
//                   the tokens' order), scaled by the pair's weight
// Tiles of 32 places x 64 weight rows; a tile lies inside one expert's group (groups are
// walked tile by tile: the grid has an upper bound of tiles, ceil(P / 32) + experts).
// Arithmetic on the CUDA cores in 32-bit; operands of the engine's type.
//
// `moe_combine`: out[m] = sum_j z[m * top + j], summed in the order of j.
//
// The expert's activation (ACT_CLAMPED_SWISH): g' = min(g, limit), u' = clamp(u, -limit, limit),
// y = g' * sigmoid(alpha * g') * (u' + shift).  (limit = infinity, alpha = 1, shift = 0: silu(g) * u.)
// `relu2` (the dense feed-forward's activation, x -> max(x, 0)^2) is here as well.
#include "common.cuh"

namespace {

constexpr int RT_THREADS = 1024;

__global__ void moe_route_table_kernel(const int* __restrict__ ids, const int* __restrict__ table, int vocab, int top,
                                       int n_experts, int M, int* __restrict__ perm, int* __restrict__ off,
                                       int* __restrict__ pair_expert) {
    ti_pdl_trigger();
    extern __shared__ int cnt[];         // [n_experts] counts, then [n_experts + 1] offsets, then [n_experts] cursors
    int* offs = cnt + n_experts;
    int* cur = offs + n_experts + 1;
    ti_pdl_sync();
    ids = ti_dependent(ids);
    const int P = M * top;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int m = p / top, j = p - m * top;
        int id = ids[m];
        id = min(max(id, 0), vocab - 1);
        int e = table[(size_t)id * top + j];
        e = min(max(e, 0), n_experts - 1);
        pair_expert[p] = e;
        atomicAdd(&cnt[e], 1);
    }
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

constexpr int GM = 32, GN = 64, GK = 32, G_THREADS = 256;

enum { ACT_NONE = 0, ACT_CLAMPED_SWISH = 1 };

// A: rows of `a` ([*, K], row stride lda); row of place i is a[(GATHER ? perm[i] / top : i)].
// W: [n_experts, N, K] (and W2 of the same shape when PAIR: the up matrix beside the gate matrix).
// out: PAIR -> y[i, n] = act(gate, up);  else z[(SCATTER ? perm[i] : i), n] = product * scale.
template <typename T, bool PAIR>
__global__ void __launch_bounds__(G_THREADS)
moe_grouped_kernel(const T* __restrict__ a, long long lda, const T* __restrict__ W, const T* __restrict__ W2,
                   T* __restrict__ out, long long ldo, const int* __restrict__ perm, const int* __restrict__ off,
                   int n_experts, int N, int K, int top, int gather, int scatter, float scale, float limit, float alpha, float shift,
                   long long w_estride) {
    ti_pdl_trigger();
    __shared__ float As[GK][GM + 1];
    __shared__ float Ws[GK][GN + 1];
    __shared__ float W2s[PAIR ? GK : 1][GN + 1];
    __shared__ int rows[GM];
    __shared__ int where[3];             // expert, first place, places in the tile
    ti_pdl_sync();
    a = ti_dependent(a); perm = ti_dependent(perm); off = ti_dependent(off);
    if (threadIdx.x == 0) {
        // tile blockIdx.x of the walk over the groups
        int t = blockIdx.x, e = 0, found = -1, first = 0, cnt = 0;
        for (; e < n_experts; e++) {
            const int lo = off[e], hi = off[e + 1];
            const int tiles = (hi - lo + GM - 1) / GM;
            if (t < tiles) { found = e; first = lo + t * GM; cnt = min(GM, hi - first); break; }
            t -= tiles;
        }
        where[0] = found; where[1] = first; where[2] = cnt;
    }
    __syncthreads();
    const int e = where[0], first = where[1], cnt = where[2];
    if (e < 0) return;
    const int n0 = blockIdx.y * GN;
    if (threadIdx.x < GM) {
        const int i = first + threadIdx.x;
        int r = -1;
        if (threadIdx.x < cnt) r = gather ? perm[i] / top : i;
        rows[threadIdx.x] = r;
    }
    __syncthreads();
    const T* We = W + (size_t)e * w_estride;
    const T* W2e = PAIR ? W2 + (size_t)e * w_estride : nullptr;
    // thread (ty, tx): places ty, ty + 8, ty + 16, ty + 24; weight rows tx, tx + 32
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    float acc[4][2], acc2[4][2];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 2; j++) { acc[i][j] = 0.f; acc2[i][j] = 0.f; }
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int idx = threadIdx.x; idx < GM * GK; idx += G_THREADS) {
            const int r = idx / GK, kk = idx - r * GK;
            const int src = rows[r];
            As[kk][r] = (src >= 0 && k0 + kk < K) ? to_f32(a[(size_t)src * lda + k0 + kk]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < GN * GK; idx += G_THREADS) {
            const int r = idx / GK, kk = idx - r * GK;
            const bool ok = n0 + r < N && k0 + kk < K;
            Ws[kk][r] = ok ? to_f32(We[(size_t)(n0 + r) * K + k0 + kk]) : 0.f;
            if constexpr (PAIR) W2s[kk][r] = ok ? to_f32(W2e[(size_t)(n0 + r) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < GK; kk++) {
            float av[4], wv[2], w2v[2];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[kk][ty + 8 * i];
#pragma unroll
            for (int j = 0; j < 2; j++) { wv[j] = Ws[kk][tx + 32 * j]; w2v[j] = PAIR ? W2s[kk][tx + 32 * j] : 0.f; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
                    if constexpr (PAIR) acc2[i][j] = fmaf(av[i], w2v[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = ty + 8 * i;
        if (r >= cnt) continue;
        const int place = first + r;
        const size_t orow = scatter ? (size_t)perm[place] : (size_t)place;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int n = n0 + tx + 32 * j;
            if (n >= N) continue;
            float y;
            if constexpr (PAIR) {
                // the two products are rounded to the engine's type first, as a kernel after the product would find them
                const float g = fminf(to_f32(from_f32<T>(acc[i][j])), limit);
                const float u = fminf(fmaxf(to_f32(from_f32<T>(acc2[i][j])), -limit), limit);
                y = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift);
            } else {
                y = acc[i][j] * scale;
            }
            out[orow * ldo + n] = from_f32<T>(y);
        }
    }
}

// The same product for bfloat16 on the tensor cores: `mma.sync m16n8k16` with float32 accumulation.  Tiles of 32 places x
// 128 weight rows, contraction in steps of 64; 8 warps as 2 (places) x 4 (weight rows), a warp 16 x 32.  The tiles of the
// next step are fetched into registers while this step's are multiplied.  Rows in shared memory are padded by 16 bytes, so
// that the eight rows a fragment load touches fall into different banks.  Needs K, lda and the matrices' rows in multiples of
// 8 elements (16-byte loads).  With MI = 2 a tile has 64 places (a warp 32 x 32): every weight fragment then feeds two
// multiplications, which is what the shared memory's bandwidth allows the tensor cores; groups of few places take MI = 1.
constexpr int TN = 128, TK = 64, T_THREADS = 256, T_LD = TK + 8;

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool PAIR, int MI>
__global__ void __launch_bounds__(T_THREADS)
moe_grouped_mma_kernel(const bf16* __restrict__ a, long long lda, const bf16* __restrict__ W, const bf16* __restrict__ W2,
                       bf16* __restrict__ out, long long ldo, const int* __restrict__ perm, const int* __restrict__ off,
                       int n_experts, int N, int K, int top, int gather, int scatter, float scale, float limit, float alpha, float shift,
                       long long w_estride) {
    ti_pdl_trigger();
    constexpr int TM = 32 * MI;
    __shared__ __align__(16) bf16 As[TM][T_LD];
    __shared__ __align__(16) bf16 Ws[TN][T_LD];
    __shared__ __align__(16) bf16 W2s[PAIR ? TN : 1][T_LD];
    __shared__ int rows[TM];
    __shared__ int where[3];
    ti_pdl_sync();
    a = ti_dependent(a); perm = ti_dependent(perm); off = ti_dependent(off);
    if (threadIdx.x == 0) {
        int t = blockIdx.x, e = 0, found = -1, first = 0, cnt = 0;
        for (; e < n_experts; e++) {
            const int lo = off[e], hi = off[e + 1];
            const int tiles = (hi - lo + TM - 1) / TM;
            if (t < tiles) { found = e; first = lo + t * TM; cnt = min(TM, hi - first); break; }
            t -= tiles;
        }
        where[0] = found; where[1] = first; where[2] = cnt;
    }
    __syncthreads();
    const int e = where[0], first = where[1], cnt = where[2];
    if (e < 0) return;
    const int n0 = blockIdx.y * TN;
    if (threadIdx.x < TM) {
        const int i = first + threadIdx.x;
        rows[threadIdx.x] = threadIdx.x < cnt ? (gather ? perm[i] / top : i) : -1;
    }
    __syncthreads();
    const bf16* We = W + (size_t)e * w_estride;
    const bf16* W2e = PAIR ? W2 + (size_t)e * w_estride : nullptr;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;             // the warp's 16 * MI places and 32 weight rows
    const int g = lane >> 2, t4 = lane & 3;
    // what this thread fetches per step: one 16-byte piece of the places' tile, four of each weight tile
    const int ar = tid >> 3, ac = (tid & 7) * 8;
    int a_src[MI];
#pragma unroll
    for (int i = 0; i < MI; i++) a_src[i] = rows[ar + 32 * i];
    uint4 ra[MI], rw[4], rw2[4];
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < MI; i++)
            ra[i] = (a_src[i] >= 0 && k0 + ac < K) ? *reinterpret_cast<const uint4*>(a + (size_t)a_src[i] * lda + k0 + ac) : zero;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = (tid >> 3) + 32 * i;
            const bool ok = n0 + r < N && k0 + ac < K;
            rw[i] = ok ? *reinterpret_cast<const uint4*>(We + (size_t)(n0 + r) * K + k0 + ac) : zero;
            if constexpr (PAIR) rw2[i] = ok ? *reinterpret_cast<const uint4*>(W2e + (size_t)(n0 + r) * K + k0 + ac) : zero;
        }
    };
    float acc[MI][4][4], acc2[MI][PAIR ? 4 : 1][4];
#pragma unroll
    for (int m = 0; m < MI; m++)
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) { acc[m][i][j] = 0.f; if constexpr (PAIR) acc2[m][i][j] = 0.f; }
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += TK) {
        __syncthreads();             // the last step's reads of the tiles are over
#pragma unroll
        for (int i = 0; i < MI; i++) *reinterpret_cast<uint4*>(&As[ar + 32 * i][ac]) = ra[i];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            *reinterpret_cast<uint4*>(&Ws[(tid >> 3) + 32 * i][ac]) = rw[i];
            if constexpr (PAIR) *reinterpret_cast<uint4*>(&W2s[(tid >> 3) + 32 * i][ac]) = rw2[i];
        }
        __syncthreads();
        if (k0 + TK < K) fetch(k0 + TK);
#pragma unroll
        for (int kk = 0; kk < TK; kk += 16) {
            uint32_t af[MI][4];
#pragma unroll
            for (int m = 0; m < MI; m++) {
                const int r0 = (wm * MI + m) * 16 + g;
                af[m][0] = *reinterpret_cast<const uint32_t*>(&As[r0][kk + 2 * t4]);
                af[m][1] = *reinterpret_cast<const uint32_t*>(&As[r0 + 8][kk + 2 * t4]);
                af[m][2] = *reinterpret_cast<const uint32_t*>(&As[r0][kk + 2 * t4 + 8]);
                af[m][3] = *reinterpret_cast<const uint32_t*>(&As[r0 + 8][kk + 2 * t4 + 8]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int n = wn * 32 + j * 8 + g;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&Ws[n][kk + 2 * t4]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&Ws[n][kk + 2 * t4 + 8]);
#pragma unroll
                for (int m = 0; m < MI; m++) mma_16816(acc[m][j], af[m], b0, b1);
                if constexpr (PAIR) {
                    const uint32_t c0 = *reinterpret_cast<const uint32_t*>(&W2s[n][kk + 2 * t4]);
                    const uint32_t c1 = *reinterpret_cast<const uint32_t*>(&W2s[n][kk + 2 * t4 + 8]);
#pragma unroll
                    for (int m = 0; m < MI; m++) mma_16816(acc2[m][j], af[m], c0, c1);
                }
            }
        }
    }
    // accumulator j: places g (elements 0, 1) and g + 8 (elements 2, 3) of the warp's 16, weight rows j * 8 + 2 t4, + 1
#pragma unroll
    for (int m = 0; m < MI; m++)
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int r = (wm * MI + m) * 16 + g + 8 * half;
        if (r >= cnt) continue;
        const int place = first + r;
        const size_t orow = scatter ? (size_t)perm[place] : (size_t)place;
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int n = n0 + wn * 32 + j * 8 + 2 * t4 + c;
                if (n >= N) continue;
                float y;
                if constexpr (PAIR) {
                    const float gt = fminf(to_f32(from_f32<bf16>(acc[m][j][2 * half + c])), limit);
                    const float u = fminf(fmaxf(to_f32(from_f32<bf16>(acc2[m][j][2 * half + c])), -limit), limit);
                    y = gt * (1.0f / (1.0f + expf(-alpha * gt))) * (u + shift);
                } else {
                    y = acc[m][j][2 * half + c] * scale;
                }
                out[orow * ldo + n] = from_f32<bf16>(y);
            }
    }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ z, T* __restrict__ out, int H, int top) {
    ti_pdl_trigger();
    ti_pdl_sync();
    z = ti_dependent(z);
    const size_t m = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; j++) s += to_f32(z[(m * top + j) * H + i]);
        out[m * H + i] = from_f32<T>(s);
    }
}

// For the tcgen05 grouped product: every expert's places padded to whole tiles of 128.  pad_src[i] is the token row that
// padded place i takes its input from (-1: a padding row), pad_of_pair[p] the padded place of pair p, tile_group[t] the
// expert of tile t (-1: none).  One block.
__global__ void moe_pad_plan_kernel(const int* __restrict__ perm, const int* __restrict__ off, int n_experts, int P, int top,
                                    int rows, int* __restrict__ pad_src, int* __restrict__ pad_of_pair, int* __restrict__ tile_group) {
    ti_pdl_trigger();
    extern __shared__ int poff[];        // [n_experts + 1] padded offsets
    ti_pdl_sync();
    perm = ti_dependent(perm); off = ti_dependent(off);
    if (threadIdx.x == 0) {
        int a = 0;
        for (int e = 0; e < n_experts; e++) { poff[e] = a; a += (off[e + 1] - off[e] + 127) / 128 * 128; }
        poff[n_experts] = a;
    }
    for (int i = threadIdx.x; i < rows; i += blockDim.x) pad_src[i] = -1;
    __syncthreads();
    for (int t = threadIdx.x; t < rows / 128; t += blockDim.x) {
        int g = -1;
        for (int e = 0; e < n_experts; e++)
            if (t * 128 >= poff[e] && t * 128 < poff[e + 1]) { g = e; break; }
        tile_group[t] = g;
    }
    for (int e = 0; e < n_experts; e++) {
        const int lo = off[e], cnt = off[e + 1] - lo;
        for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
            const int p = perm[lo + i], at = poff[e] + i;
            pad_src[at] = p / top;
            pad_of_pair[p] = at;
        }
    }
}

template <typename T>
__global__ void moe_gather_rows_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ pad_src, T* __restrict__ xs, int H) {
    ti_pdl_trigger();
    ti_pdl_sync();
    x = ti_dependent(x); pad_src = ti_dependent(pad_src);
    const size_t i = blockIdx.x;
    const int src = pad_src[i];
    if ((H & 7) == 0 && sizeof(T) == 2) {
        const uint4* s4 = src >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)src * ldx) : nullptr;
        uint4* d4 = reinterpret_cast<uint4*>(xs + i * H);
        for (int e = threadIdx.x; e < H / 8; e += blockDim.x) d4[e] = s4 ? s4[e] : make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (int e = threadIdx.x; e < H; e += blockDim.x) xs[i * H + e] = src >= 0 ? x[(size_t)src * ldx + e] : from_f32<T>(0.f);
    }
}

// the same over 16-byte pieces of bfloat16 (ff a multiple of 8)
__global__ void moe_act_pair_vec_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y, int ff8, long long total, float limit, float alpha, float shift) {
    ti_pdl_trigger();
    ti_pdl_sync();
    gu = ti_dependent(gu);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long i = idx / ff8;
        const int c = (int)(idx - i * ff8);
        const uint4 g4 = reinterpret_cast<const uint4*>(gu)[i * 2 * ff8 + c], u4 = reinterpret_cast<const uint4*>(gu)[i * 2 * ff8 + ff8 + c];
        const bf16* gp = reinterpret_cast<const bf16*>(&g4);
        const bf16* up = reinterpret_cast<const bf16*>(&u4);
        uint4 o4;
        bf16* op = reinterpret_cast<bf16*>(&o4);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float g = fminf(to_f32(gp[e]), limit);
            const float u = fminf(fmaxf(to_f32(up[e]), -limit), limit);
            op[e] = from_f32<bf16>(g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift));
        }
        reinterpret_cast<uint4*>(y)[idx] = o4;
    }
}

// the squared ReLU over 16-byte pieces of bfloat16
__global__ void relu2_vec_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, long long n8) {
    ti_pdl_trigger();
    ti_pdl_sync();
    x = ti_dependent(x);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const uint4 v4 = reinterpret_cast<const uint4*>(x)[i];
        const bf16* vp = reinterpret_cast<const bf16*>(&v4);
        uint4 o4;
        bf16* op = reinterpret_cast<bf16*>(&o4);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float v = fmaxf(to_f32(vp[e]), 0.f);
            op[e] = from_f32<bf16>(v * v);
        }
        reinterpret_cast<uint4*>(out)[i] = o4;
    }
}

// gu[i] = [gate (ff) | up (ff)] -> y[i] = g' sigmoid(alpha g') (u' + shift)
template <typename T>
__global__ void moe_act_pair_kernel(const T* __restrict__ gu, T* __restrict__ y, int ff, long long total, float limit, float alpha, float shift) {
    ti_pdl_trigger();
    ti_pdl_sync();
    gu = ti_dependent(gu);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long i = idx / ff;
        const int f = (int)(idx - i * ff);
        const float g = fminf(to_f32(gu[i * 2 * ff + f]), limit);
        const float u = fminf(fmaxf(to_f32(gu[i * 2 * ff + ff + f]), -limit), limit);
        y[idx] = from_f32<T>(g * (1.0f / (1.0f + expf(-alpha * g))) * (u + shift));
    }
}

// out[m] = sum_j z[pad_of_pair[m * top + j]] * weight, each term rounded as the scattering product would have stored it
template <typename T>
__global__ void moe_combine_indexed_kernel(const T* __restrict__ z, const int* __restrict__ pad_of_pair, T* __restrict__ out, int H,
                                           int top, float weight) {
    ti_pdl_trigger();
    ti_pdl_sync();
    z = ti_dependent(z); pad_of_pair = ti_dependent(pad_of_pair);
    const size_t m = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; j++) {
            const float term = to_f32(from_f32<T>(to_f32(z[(size_t)pad_of_pair[m * top + j] * H + i]) * weight));
            s = j == 0 ? term : s + term;
        }
        out[m * H + i] = from_f32<T>(s);
    }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
    ti_pdl_trigger();
    ti_pdl_sync();
    x = ti_dependent(x);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(x[i]), 0.f);
        out[i] = from_f32<T>(v * v);
    }
}

}  // namespace

// ids: int32 [M]; table: int32 [vocab, top]; perm: int32 [M * top]; off: int32 [n_experts + 1];
// pair_expert: int32 scratch [M * top].
extern "C" int ti_moe_route_table(const int* ids, const int* table, int vocab, int top, int n_experts, int M, int* perm,
                                  int* off, int* pair_expert, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && top > 0 && n_experts > 0 && vocab > 0, "moe_route_table: bad sizes");
    const size_t smem = (size_t)(3 * n_experts + 1) * sizeof(int);
    TI_REQUIRE(smem <= 48 * 1024, "moe_route_table: %d experts are too many", n_experts);
    TI_CUDA(ti_launch_class<1>(moe_route_table_kernel, dim3(1), dim3(RT_THREADS), smem, stream, ids, table, vocab, top, n_experts, M,
                               perm, off, pair_expert));
    TI_CHECK_LAUNCH("moe_route_table");
    return 0;
}

// P places.  pair != 0: out[i, 0:N] = act(a_i W[e]^T, a_i W2[e]^T).  Else out[(scatter ? perm[i] : i)] = a_i W[e]^T * scale.
extern "C" int ti_moe_grouped(const void* a, long long lda, const void* W, const void* W2, void* out, long long ldo,
                              const int* perm, const int* off, int n_experts, int P, int N, int K, int top, int gather,
                              int scatter, int pair, float scale, float limit, float alpha, float shift, long long w_estride, int dtype,
                              cudaStream_t stream) {
    if (P == 0) return 0;
    if (w_estride <= 0) w_estride = (long long)N * K;          // elements from one expert's matrix to the next
    TI_REQUIRE(P > 0 && N > 0 && K > 0 && n_experts > 0 && top > 0, "moe_grouped: bad sizes");
    TI_REQUIRE(!pair || W2, "moe_grouped: the paired form needs a second matrix");
    const bool tensor_cores = dtype == TI_BF16 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)W & 15) == 0 &&
                              (!W2 || ((uintptr_t)W2 & 15) == 0);
    if (tensor_cores) {
        const bool big = P >= 48 * n_experts;         // groups of 48 places and more on average: tiles of 64
        const int tm = big ? 64 : 32;
        const int tiles = (P + tm - 1) / tm + n_experts;
        const int nblk = (N + TN - 1) / TN;
        TI_REQUIRE(nblk <= 65535, "moe_grouped: %d weight rows are too many for one launch", N);
#define TI_MOE_LAUNCH(PAIR, MI) TI_CUDA(ti_launch(moe_grouped_mma_kernel<PAIR, MI>, dim3(tiles, nblk), dim3(T_THREADS), 0, stream, (const bf16*)a, lda, \
                              (const bf16*)W, (const bf16*)W2, (bf16*)out, ldo, perm, off, n_experts, N, K, top, gather, scatter, scale, limit, alpha, shift, w_estride))
        if (pair) { if (big) TI_MOE_LAUNCH(true, 2); else TI_MOE_LAUNCH(true, 1); }
        else { if (big) TI_MOE_LAUNCH(false, 2); else TI_MOE_LAUNCH(false, 1); }
#undef TI_MOE_LAUNCH
        TI_CHECK_LAUNCH("moe_grouped");
        return 0;
    }
    const int tiles = (P + GM - 1) / GM + n_experts;
    const int nblk = (N + GN - 1) / GN;
    TI_REQUIRE(nblk <= 65535, "moe_grouped: %d weight rows are too many for one launch", N);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        if (pair)
            TI_CUDA(ti_launch(moe_grouped_kernel<T, true>, dim3(tiles, nblk), dim3(G_THREADS), 0, stream, (const T*)a, lda,
                              (const T*)W, (const T*)W2, (T*)out, ldo, perm, off, n_experts, N, K, top, gather, scatter, scale, limit, alpha, shift, w_estride));
        else
            TI_CUDA(ti_launch(moe_grouped_kernel<T, false>, dim3(tiles, nblk), dim3(G_THREADS), 0, stream, (const T*)a, lda,
                              (const T*)W, (const T*)W2, (T*)out, ldo, perm, off, n_experts, N, K, top, gather, scatter, scale, limit, alpha, shift, w_estride));
        TI_CHECK_LAUNCH("moe_grouped");
        return 0;
    });
}

extern "C" int ti_moe_combine(const void* z, void* out, int M, int H, int top, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && H > 0 && top > 0, "moe_combine: bad sizes");
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(moe_combine_kernel<T>, dim3(M), dim3(H <= 256 ? 64 : 256), 0, stream, (const T*)z, (T*)out, H, top));
        TI_CHECK_LAUNCH("moe_combine");
        return 0;
    });
}

extern "C" int ti_moe_pad_plan(const int* perm, const int* off, int n_experts, int P, int top, int rows, int* pad_src,
                               int* pad_of_pair, int* tile_group, cudaStream_t stream) {
    if (P == 0) return 0;
    TI_REQUIRE(P > 0 && n_experts > 0 && top > 0 && rows % 128 == 0 && rows >= P + 0, "moe_pad_plan: bad sizes");
    const size_t smem = (size_t)(n_experts + 1) * sizeof(int);
    TI_REQUIRE(smem <= 48 * 1024, "moe_pad_plan: %d experts are too many", n_experts);
    TI_CUDA(ti_launch_class<1>(moe_pad_plan_kernel, dim3(1), dim3(1024), smem, stream, perm, off, n_experts, P, top, rows, pad_src,
                               pad_of_pair, tile_group));
    TI_CHECK_LAUNCH("moe_pad_plan");
    return 0;
}

extern "C" int ti_moe_gather_rows(const void* x, long long ldx, const int* pad_src, void* xs, int rows, int H, int dtype,
                                  cudaStream_t stream) {
    if (rows == 0) return 0;
    TI_REQUIRE(rows > 0 && H > 0, "moe_gather_rows: bad sizes");
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_REQUIRE(sizeof(T) != 2 || (H & 7) || ((((uintptr_t)x | (uintptr_t)xs) & 15) == 0 && ldx % 8 == 0),
                   "moe_gather_rows: rows are not 16-byte aligned");
        TI_CUDA(ti_launch_class<1>(moe_gather_rows_kernel<T>, dim3(rows), dim3(128), 0, stream, (const T*)x, ldx, pad_src, (T*)xs, H));
        TI_CHECK_LAUNCH("moe_gather_rows");
        return 0;
    });
}

extern "C" int ti_moe_act_pair(const void* gu, void* y, long long rows, int ff, float limit, float alpha, float shift, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    TI_REQUIRE(rows > 0 && ff > 0, "moe_act_pair: bad sizes");
    if (dtype == TI_BF16 && ff % 8 == 0 && (((uintptr_t)gu | (uintptr_t)y) & 15) == 0) {
        const long long n = rows * (ff / 8);
        const long long want = (n + 255) / 256;
        TI_CUDA(ti_launch_class<1>(moe_act_pair_vec_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, stream,
                                   (const bf16*)gu, (bf16*)y, ff / 8, n, limit, alpha, shift));
        TI_CHECK_LAUNCH("moe_act_pair");
        return 0;
    }
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const long long n = rows * ff;
        const long long want = (n + 255) / 256;
        TI_CUDA(ti_launch_class<1>(moe_act_pair_kernel<T>, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, stream,
                                   (const T*)gu, (T*)y, ff, n, limit, alpha, shift));
        TI_CHECK_LAUNCH("moe_act_pair");
        return 0;
    });
}

extern "C" int ti_moe_combine_indexed(const void* z, const int* pad_of_pair, void* out, int M, int H, int top, float weight, int dtype,
                                      cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && H > 0 && top > 0, "moe_combine_indexed: bad sizes");
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(moe_combine_indexed_kernel<T>, dim3(M), dim3(H <= 256 ? 64 : 256), 0, stream, (const T*)z, pad_of_pair,
                                   (T*)out, H, top, weight));
        TI_CHECK_LAUNCH("moe_combine_indexed");
        return 0;
    });
}

extern "C" int ti_relu2(const void* x, void* out, long long n, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(n > 0, "relu2: bad size");
    if (dtype == TI_BF16 && n % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        const long long n8 = n / 8, want = (n8 + 255) / 256;
        TI_CUDA(ti_launch_class<1>(relu2_vec_kernel, dim3((unsigned)(want < 148 * 16 ? want : 148 * 16)), dim3(256), 0, stream,
                                   (const bf16*)x, (bf16*)out, n8));
        TI_CHECK_LAUNCH("relu2");
        return 0;
    }
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const int threads = 256;
        const long long want = (n + threads - 1) / threads;
        const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
        TI_CUDA(ti_launch_class<1>(relu2_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (const T*)x, (T*)out, n));
        TI_CHECK_LAUNCH("relu2");
        return 0;
    });
}
