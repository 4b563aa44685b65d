// Linear attention with a per-head decay ("lightning" attention) and the gated norm after it.
//
// Per head, with a state S [dim, vdim] in float32 that a sequence carries from token to token
// (zero when the sequence starts):
//     S_t = decay_h * S_{t-1} + k_t v_t^T,      o_t = S_t^T q_t
// where q, k, v are the projections' outputs after the entry function (`act` 1: silu,
// z / (1 + exp(-z)); 0: as they are), applied here as the values are loaded, and k is then
// multiplied by `k_scale` (a retention layer's dim^(-1/2); 1 otherwise).  Everything of the
// recurrence is 32-bit.
//
// lightning_scan: a sequence's new tokens are scanned in order from the state in its slot,
// which is updated in place: whole prompts, single tokens and anything between are one
// kernel.  Grid (heads * column groups, sequences): a thread owns one column of S
// (dim registers) and needs no other thread's work; q and k of a run of tokens are staged in
// shared memory.
//
// lightning_chunk_*: the same for long runs of new tokens, in three kernels that work on
// chunks of C tokens in parallel: (1) every chunk's own contribution
// U_c = sum_s decay^(C-1-s) k_s v_s^T, (2) the states before every chunk by a scan over the
// chunks, S_c = decay^C S_{c-1} + U_c, (3) every token's output from the state before its
// chunk and the tokens of the chunk up to itself,
// o_t = decay^(t+1) S^T q_t + sum_{s<=t} decay^(t-s) (q_t . k_s) v_s.
//
// gated_rmsnorm: y = rms(o) * w * sigmoid(g) over all heads' outputs of a token together.
#include "common.cuh"

#include <type_traits>

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// what q, k and v pass as they enter the recurrence
struct Entry { int act; float k_scale; };
__device__ __forceinline__ float enter(float z, int act) { return act ? silu_f(z) : z; }

constexpr int SCAN_TOK = 16;     // tokens staged at a time

template <typename T, int MAXD>
__global__ void lightning_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                      long long q_stride, long long k_stride, long long v_stride,
                                      float* __restrict__ o, float* __restrict__ state, const float* __restrict__ decay,
                                      const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                                      int n_heads, int dim, int vdim, int groups, Entry en) {
    ti_pdl_trigger();
    extern __shared__ float sm[];        // q: [SCAN_TOK][dim], k: [SCAN_TOK][dim]
    ti_pdl_sync();
    q = ti_dependent(q); k = ti_dependent(k); v = ti_dependent(v);
    float* qs = sm;
    float* ks = sm + SCAN_TOK * dim;
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    const int b = blockIdx.y;
    const int tok0 = cu_new[b], n = cu_new[b + 1] - tok0;
    if (n <= 0) return;
    const int slot = seq_slot[b];
    const int col = g * blockDim.x + threadIdx.x;
    const bool live = col < vdim;
    const float lam = decay[h];
    float S[MAXD];
    float* srow = state + ((size_t)slot * n_heads + h) * dim * vdim;
#pragma unroll
    for (int i = 0; i < MAXD; i++) S[i] = (live && i < dim) ? srow[(size_t)i * vdim + col] : 0.f;
    for (int t0 = 0; t0 < n; t0 += SCAN_TOK) {
        const int nt = min(SCAN_TOK, n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * dim; idx += blockDim.x) {
            const int tt = idx / dim, i = idx - tt * dim;
            const size_t tok = (size_t)(tok0 + t0 + tt);
            qs[idx] = enter(to_f32(q[tok * q_stride + (size_t)h * dim + i]), en.act);
            ks[idx] = enter(to_f32(k[tok * k_stride + (size_t)h * dim + i]), en.act) * en.k_scale;
        }
        __syncthreads();
        if (live) {
            for (int tt = 0; tt < nt; tt++) {
                const size_t tok = (size_t)(tok0 + t0 + tt);
                const float vv = enter(to_f32(v[tok * v_stride + (size_t)h * vdim + col]), en.act);
                const float* kr = ks + tt * dim;
                const float* qr = qs + tt * dim;
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < MAXD; i++) {
                    if (i < dim) {
                        S[i] = fmaf(lam, S[i], kr[i] * vv);
                        acc = fmaf(S[i], qr[i], acc);
                    }
                }
                o[tok * ((size_t)n_heads * vdim) + (size_t)h * vdim + col] = acc;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < MAXD; i++)
            if (i < dim) srow[(size_t)i * vdim + col] = S[i];
    }
}

// ---------------------------------------------------------------------------
// chunked form
// ---------------------------------------------------------------------------
constexpr int CH = 64;           // tokens per chunk

// chunk c of sequence b covers its new tokens [c * CH, min(n, (c + 1) * CH)); chunk_of[b] is the index of
// the sequence's first chunk among all chunks of the step (a prefix sum of ceil(n / CH)).
struct Chunks { const int* cu_new; const int* seq_slot; int n_seq; };

__device__ __forceinline__ bool find_chunk(const Chunks& cz, int chunk, int& b, int& c, int& tok0, int& n) {
    // a linear walk over the sequences: steps have few of them
    int seen = 0;
    for (int s = 0; s < cz.n_seq; s++) {
        const int a = cz.cu_new[s], len = cz.cu_new[s + 1] - a;
        const int nchunks = (len + CH - 1) / CH;
        if (chunk < seen + nchunks) { b = s; c = chunk - seen; tok0 = a; n = len; return true; }
        seen += nchunks;
    }
    return false;
}

// The chunk kernels are small matrix products on the CUDA cores in 32-bit, operands in shared memory, a thread a tile of
// the result in registers.  Column groups of 128: grid.x = heads * groups.
constexpr int CT = 256;          // threads of a chunk kernel
constexpr int VG = 128;          // value columns per block

// (1) U[chunk, h][i][j] = sum_s lam^(nt-1-s) k_s[i] v_s[j] over the chunk's nt tokens: a [dim x nt] x [nt x VG] product.
// Thread (ty, tx) of 16 x 16: rows i = ty + 16 a (a < 8), columns j = 8 tx .. 8 tx + 7.
template <typename T>
__global__ void __launch_bounds__(CT)
lightning_chunk_local_kernel(const T* __restrict__ k, const T* __restrict__ v, long long k_stride, long long v_stride,
                             float* __restrict__ U, const float* __restrict__ decay, Chunks cz, int n_heads, int dim,
                             int vdim, int groups, Entry en) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    float* ks = sm;                      // [CH][128]  (lam^(nt-1-s) k_s, zero past dim)
    float* vs = ks + CH * 128;           // [CH][VG]
    __shared__ float pw[CH];             // lam^(nt-1-s)
    ti_pdl_sync();
    k = ti_dependent(k); v = ti_dependent(v);
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    int b, c, tok0, n;
    if (!find_chunk(cz, blockIdx.y, b, c, tok0, n)) return;
    const int t0 = c * CH, nt = min(CH, n - t0), j0 = g * VG;
    const float lam = decay[h];
    if (threadIdx.x < CH) pw[threadIdx.x] = threadIdx.x < nt ? powf(lam, (float)(nt - 1 - (int)threadIdx.x)) : 0.f;
    __syncthreads();
    // (loads in batches of 8, so that eight are on their way at a time: a block's few warps cannot hide one load each)
    for (int it = 0; it < CH * 128 / CT; it += 8) {
        float x[8], y[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = (it + u) * CT + threadIdx.x, tt = idx >> 7, i = idx & 127;
            x[u] = (tt < nt && i < dim) ? to_f32(k[(size_t)(tok0 + t0 + tt) * k_stride + (size_t)h * dim + i]) : 0.f;
            y[u] = (tt < nt && j0 + i < vdim) ? to_f32(v[(size_t)(tok0 + t0 + tt) * v_stride + (size_t)h * vdim + j0 + i]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = (it + u) * CT + threadIdx.x, tt = idx >> 7, i = idx & 127;
            ks[idx] = (tt < nt && i < dim) ? enter(x[u], en.act) * en.k_scale * pw[tt] : 0.f;
            vs[idx] = (tt < nt && j0 + i < vdim) ? enter(y[u], en.act) : 0.f;
        }
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; a++)
#pragma unroll
        for (int e = 0; e < 8; e++) acc[a][e] = 0.f;
    for (int tt = 0; tt < nt; tt++) {
        float kv[8], vv[8];
#pragma unroll
        for (int a = 0; a < 8; a++) kv[a] = ks[tt * 128 + ty + 16 * a];
        const float4 v0 = *reinterpret_cast<const float4*>(vs + tt * VG + 8 * tx), v1 = *reinterpret_cast<const float4*>(vs + tt * VG + 8 * tx + 4);
        vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
#pragma unroll
        for (int a = 0; a < 8; a++)
#pragma unroll
            for (int e = 0; e < 8; e++) acc[a][e] = fmaf(kv[a], vv[e], acc[a][e]);
    }
    float* u = U + ((size_t)blockIdx.y * n_heads + h) * dim * vdim;
#pragma unroll
    for (int a = 0; a < 8; a++) {
        const int i = ty + 16 * a;
        if (i >= dim) continue;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int j = j0 + 8 * tx + e;
            if (j < vdim) u[(size_t)i * vdim + j] = acc[a][e];
        }
    }
}

// (2) per sequence and head, over its chunks in order: U[chunk] <- state before the chunk, state <- state after the
// last chunk.  One thread per element of the state.
__global__ void lightning_chunk_scan_kernel(float* __restrict__ U, float* __restrict__ state, const float* __restrict__ decay,
                                            Chunks cz, int n_heads, int dim, int vdim) {
    ti_pdl_trigger();
    ti_pdl_sync();
    const int b = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= dim * vdim) return;
    int first = 0;
    for (int s = 0; s < b; s++) first += (cz.cu_new[s + 1] - cz.cu_new[s] + CH - 1) / CH;
    const int n = cz.cu_new[b + 1] - cz.cu_new[b];
    if (n <= 0) return;
    const int nchunks = (n + CH - 1) / CH;
    const float lam = decay[h];
    const float whole = powf(lam, (float)CH), rest = powf(lam, (float)(n - (nchunks - 1) * CH));
    float* sp = state + ((size_t)cz.seq_slot[b] * n_heads + h) * dim * vdim + e;
    float* u = U + ((size_t)first * n_heads + h) * dim * vdim + e;
    const size_t step = (size_t)n_heads * dim * vdim;
    float S = *sp;
    // a chunk's own contribution is read before the state before it is stored in its place; eight reads go out together
    for (int c0 = 0; c0 < nchunks; c0 += 8) {
        float own[8];
#pragma unroll
        for (int j = 0; j < 8; j++) own[j] = c0 + j < nchunks ? u[(size_t)j * step] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (c0 + j < nchunks) {
                u[(size_t)j * step] = S;
                S = fmaf(c0 + j + 1 < nchunks ? whole : rest, S, own[j]);
            }
        }
        u += 8 * step;
    }
    *sp = S;
}

// (3) outputs of a chunk, O = diag(lam^(t+1)) Q S + A V with A[t][s] = lam^(t-s) (q_t . k_s) for s <= t, S the state before
// the chunk: A is formed first (a [nt x dim] x [dim x nt] product), then the two products add into the same registers.
// 512 threads (the operands leave room for one block per SM: sixteen warps hide more than eight): thread (ty, tx) of
// 16 x 32 has tokens t = ty + 16 a (a < 4) and columns j = 4 tx .. 4 tx + 3.
constexpr int CO = 512;

template <typename T>
__global__ void __launch_bounds__(CO)
lightning_chunk_out_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                           long long q_stride, long long k_stride, long long v_stride,
                           const float* __restrict__ U, float* __restrict__ o,
                           const float* __restrict__ decay, Chunks cz, int n_heads, int dim, int vdim, int groups, Entry en) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    q = ti_dependent(q); k = ti_dependent(k); v = ti_dependent(v); U = ti_dependent(U);
    constexpr int LDQ = 129;
    float* qs = sm;                      // [CH][129]
    float* kv = qs + CH * LDQ;           // [CH][129] keys, later [CH][VG] values
    float* A = kv + CH * LDQ;            // [CH][CH + 1]
    float* pw = A + CH * (CH + 1);       // lam^0 .. lam^CH
    float* Ss = pw + CH + 4;             // [128][VG] the state before the chunk (zero past dim)
    const int h = blockIdx.x / groups, g = blockIdx.x - h * groups;
    int b, c, tok0, n;
    if (!find_chunk(cz, blockIdx.y, b, c, tok0, n)) return;
    const int t0 = c * CH, nt = min(CH, n - t0), j0 = g * VG;
    const float lam = decay[h];
    const int tid = threadIdx.x;
    // (loads in batches of 8: see lightning_chunk_local_kernel)
    for (int it = 0; it < CH * 128 / CO; it += 8) {
        float x[8], y[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = (it + u) * CO + tid, tt = idx >> 7, i = idx & 127;
            const bool ok = tt < nt && i < dim;
            const size_t tok = (size_t)(tok0 + t0 + tt);
            x[u] = ok ? to_f32(q[tok * q_stride + (size_t)h * dim + i]) : 0.f;
            y[u] = ok ? to_f32(k[tok * k_stride + (size_t)h * dim + i]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = (it + u) * CO + tid, tt = idx >> 7, i = idx & 127;
            const bool ok = tt < nt && i < dim;
            qs[tt * LDQ + i] = ok ? enter(x[u], en.act) : 0.f;
            kv[tt * LDQ + i] = ok ? enter(y[u], en.act) * en.k_scale : 0.f;
        }
    }
    const float* Sg = U + ((size_t)blockIdx.y * n_heads + h) * dim * vdim;
    for (int it = 0; it < 128 * VG / CO; it += 8) {
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = (it + u) * CO + tid, i = idx >> 7, j = idx & 127;
            x[u] = (i < dim && j0 + j < vdim) ? Sg[(size_t)i * vdim + j0 + j] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) Ss[(it + u) * CO + tid] = x[u];
    }
    for (int i = tid; i <= CH; i += CO) pw[i] = powf(lam, (float)i);
    __syncthreads();
    const int ty = tid >> 5, tx = tid & 31;
    {   // A: tokens t = ty + 16 a (a < 4), keys s = tx + 32 e (e < 2)
        float acc[4][2];
#pragma unroll
        for (int a = 0; a < 4; a++) { acc[a][0] = 0.f; acc[a][1] = 0.f; }
        for (int i = 0; i < dim; i++) {
            float qv[4];
#pragma unroll
            for (int a = 0; a < 4; a++) qv[a] = qs[(ty + 16 * a) * LDQ + i];
            const float k0 = kv[tx * LDQ + i], k1 = kv[(tx + 32) * LDQ + i];
#pragma unroll
            for (int a = 0; a < 4; a++) { acc[a][0] = fmaf(qv[a], k0, acc[a][0]); acc[a][1] = fmaf(qv[a], k1, acc[a][1]); }
        }
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int tt = ty + 16 * a, ss = tx + 32 * e;
                A[tt * (CH + 1) + ss] = (ss <= tt && tt < nt) ? acc[a][e] * pw[tt - ss] : 0.f;
            }
    }
    __syncthreads();                     // A is whole, the keys are done with
    for (int it = 0; it < CH * VG / CO; it += 8) {
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = (it + u) * CO + tid, tt = idx >> 7, j = idx & 127;
            x[u] = (tt < nt && j0 + j < vdim) ? to_f32(v[(size_t)(tok0 + t0 + tt) * v_stride + (size_t)h * vdim + j0 + j]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = (it + u) * CO + tid, tt = idx >> 7, j = idx & 127;
            kv[idx] = (tt < nt && j0 + j < vdim) ? enter(x[u], en.act) : 0.f;
        }
    }
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[a][e] = 0.f;
    for (int i = 0; i < dim; i++) {
        float qv[4];
#pragma unroll
        for (int a = 0; a < 4; a++) qv[a] = qs[(ty + 16 * a) * LDQ + i];
        const float4 s0 = *reinterpret_cast<const float4*>(Ss + i * VG + 4 * tx);
        const float sv[4] = {s0.x, s0.y, s0.z, s0.w};
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[a][e] = fmaf(qv[a], sv[e], acc[a][e]);
    }
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[a][e] *= pw[ty + 16 * a + 1];
    __syncthreads();                     // the values are in place
    for (int ss = 0; ss < nt; ss++) {
        float av[4];
#pragma unroll
        for (int a = 0; a < 4; a++) av[a] = A[(ty + 16 * a) * (CH + 1) + ss];
        const float4 v0 = *reinterpret_cast<const float4*>(kv + ss * VG + 4 * tx);
        const float vv[4] = {v0.x, v0.y, v0.z, v0.w};
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[a][e] = fmaf(av[a], vv[e], acc[a][e]);
    }
#pragma unroll
    for (int a = 0; a < 4; a++) {
        const int tt = ty + 16 * a;
        if (tt >= nt) continue;
        float* orow = o + (size_t)(tok0 + t0 + tt) * ((size_t)n_heads * vdim) + (size_t)h * vdim;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int j = j0 + 4 * tx + e;
            if (j < vdim) orow[j] = acc[a][e];
        }
    }
}

// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ g, long long g_stride,
                                     const float* __restrict__ w, T* __restrict__ out, int N, float eps) {
    ti_pdl_trigger();
    __shared__ float red[33];
    ti_pdl_sync();
    o = ti_dependent(o); g = ti_dependent(g);
    const size_t m = blockIdx.x;
    const float* orow = o + m * N;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss = fmaf(orow[i], orow[i], ss);
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float gate = 1.0f / (1.0f + expf(-to_f32(g[m * g_stride + i])));
        out[m * N + i] = from_f32<T>(orow[i] * inv * w[i] * gate);
    }
}

template <typename F>
int dispatch_dim(int dim, F&& f) {
    if (dim <= 32) return f(std::integral_constant<int, 32>());
    if (dim <= 64) return f(std::integral_constant<int, 64>());
    if (dim <= 128) return f(std::integral_constant<int, 128>());
    ti_set_error("lightning: heads of %d query/key elements are not supported (up to 128)", dim);
    return 1;
}

int column_threads(int vdim) { return vdim <= 32 ? 32 : vdim <= 64 ? 64 : 128; }

}  // namespace

// q, k: [M, heads, dim], v: [M, heads, vdim] (token strides given), before the entry function (act 1: silu, 0: none;
// k then times k_scale).  o: float32 [M, heads * vdim].  state: float32 [slots, heads, dim, vdim].
extern "C" int ti_lightning_scan(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                 long long v_stride, float* o, float* state, const float* decay, const int* cu_new,
                                 const int* seq_slot, int n_seq, int n_heads, int dim, int vdim, int act, float k_scale,
                                 int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && n_heads > 0 && dim > 0 && vdim > 0, "lightning_scan: bad sizes");
    const int threads = column_threads(vdim), groups = (vdim + threads - 1) / threads;
    const size_t smem = (size_t)2 * SCAN_TOK * dim * sizeof(float);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        return dispatch_dim(dim, [&](auto md) -> int {
            constexpr int MAXD = decltype(md)::value;
            TI_CUDA(ti_launch(lightning_scan_kernel<T, MAXD>, dim3(n_heads * groups, n_seq), dim3(threads), smem, stream,
                              (const T*)q, (const T*)k, (const T*)v, q_stride, k_stride, v_stride, o, state, decay, cu_new,
                              seq_slot, n_heads, dim, vdim, groups, Entry{act, k_scale}));
            TI_CHECK_LAUNCH("lightning_scan");
            return 0;
        });
    });
}

// The chunked form: n_chunks >= sum over sequences of ceil(new tokens / 64) (an upper bound is enough);
// U: float32 scratch [n_chunks, heads, dim, vdim].
extern "C" int ti_lightning_chunked(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                    long long v_stride, float* o, float* state, float* U, const float* decay,
                                    const int* cu_new, const int* seq_slot, int n_seq, int n_chunks, int n_heads, int dim,
                                    int vdim, int act, float k_scale, int dtype, cudaStream_t stream) {
    if (n_seq == 0 || n_chunks == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && n_chunks > 0 && n_chunks <= 65535 && n_heads > 0 && n_heads <= 65535 && dim > 0 && vdim > 0,
               "lightning_chunked: bad sizes");
    TI_REQUIRE(dim <= 128, "lightning: heads of %d query/key elements are not supported (up to 128)", dim);
    const int groups = (vdim + VG - 1) / VG;
    Chunks cz{cu_new, seq_slot, n_seq};
    const Entry en{act, k_scale};
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const size_t smem1 = (size_t)(CH * 128 + CH * VG) * sizeof(float);
        const size_t smem3 = ((size_t)2 * CH * 129 + (size_t)CH * (CH + 1) + CH + 4 + (size_t)128 * VG) * sizeof(float);
        static bool configured = false;
        if (!configured) {
            TI_CUDA(cudaFuncSetAttribute(lightning_chunk_local_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
            TI_CUDA(cudaFuncSetAttribute(lightning_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3));
            configured = true;
        }
        TI_CUDA(ti_launch(lightning_chunk_local_kernel<T>, dim3(n_heads * groups, n_chunks), dim3(CT), smem1, stream,
                          (const T*)k, (const T*)v, k_stride, v_stride, U, decay, cz, n_heads, dim, vdim, groups, en));
        TI_CHECK_LAUNCH("lightning_chunk_local");
        TI_CUDA(ti_launch(lightning_chunk_scan_kernel, dim3((dim * vdim + 127) / 128, n_heads, n_seq), dim3(128), 0, stream,
                          U, state, decay, cz, n_heads, dim, vdim));
        TI_CHECK_LAUNCH("lightning_chunk_scan");
        TI_CUDA(ti_launch(lightning_chunk_out_kernel<T>, dim3(n_heads * groups, n_chunks), dim3(CO), smem3, stream,
                          (const T*)q, (const T*)k, (const T*)v, q_stride, k_stride, v_stride, (const float*)U, o, decay, cz,
                          n_heads, dim, vdim, groups, en));
        TI_CHECK_LAUNCH("lightning_chunk_out");
        return 0;
    });
}

// o: float32 [M, N]; g: [M, N] of the engine's type with row stride g_stride; w: float32 [N]; out: [M, N].
extern "C" int ti_gated_rmsnorm(const float* o, const void* g, long long g_stride, const float* w, void* out, int M, int N,
                                float eps, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && N > 0 && g_stride >= N, "gated_rmsnorm: bad sizes M=%d N=%d", M, N);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const int threads = N <= 256 ? 64 : N <= 1024 ? 128 : 256;
        TI_CUDA(ti_launch_class<1>(gated_rmsnorm_kernel<T>, dim3(M), dim3(threads), 0, stream, o, (const T*)g, g_stride, w, (T*)out, N, eps));
        TI_CHECK_LAUNCH("gated_rmsnorm");
        return 0;
    });
}
