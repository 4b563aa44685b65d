// Sliding-window grouped-query attention in two flavours that share their kernels, over keys and
// values of different sizes read from the paged cache.  CUDA cores, everything after the loads in
// 32-bit.
//
// A query head may carry several score MAPS (differential attention has two): head h of the
// projection's row holds `maps` queries of `dim` elements side by side, kv head g holds `maps`
// keys side by side and ONE value of `vdim` elements.  The kernels treat (head, map) as a
// virtual head hv = h * maps + map, which reads kv head h / (heads / kv_heads), the key at offset
// map * dim of that head's row, and the head's value.
//
// For the query at position i and the key at position j of a sequence, visible when
// 0 <= i - j < window (window <= 0: every j <= i), or, whatever the window, when j <= i and
// j < keep_first (a sequence's first positions stay visible to every later query, at their own
// positions); results may be multiplied by `out_scale` before they are rounded:
//     s_ij = (q_i . k_j) * scale - r1[h] * ln(1 + r2[h] * (i - j))          (r1 == null: no distance term)
//     MODE 0:  softmax over the visible j,  o_i = sum_j p_ij v_j
//     MODE 1:  w_ij = sigmoid(s_ij + pb[h]), not normalised over j,  o_i = sum_j w_ij v_j
//
// attn_window_prepare: a block per token over the projection's row [q | k | v | ...]: adds the
//   projections' biases, norms ALL of q's and ALL of k's elements at once (x * rsqrt(mean(x^2) + eps)
//   * w[i], a weight per element; each optional), rotates the first `rot` elements of every map of
//   q and k by the token's position (pairs (e, e + rot/2), tables of cos and sin), writes q, k and
//   v back in place and stores k and v at the token's position in the sequence's pages.  Where the
//   sizes and addresses allow it the row moves in runs of 16 bytes (attn_window_prepare_vec).
// attn_head_prepare: the same place in a step for a design whose norms run per head: a warp per
//   token and head over the projection's row [q | k | v | ...] (one map): adds the projections'
//   biases, norms every head of q and of k over its own `dim` elements with one weight [dim] for all
//   heads (each optional), rotates the first `rot` elements of every head of q and k, pairing either
//   (e, e + rot/2) or neighbours (2e, 2e + 1) with the same tables, writes back and stores k and v.
// attn_window: any number of new tokens per sequence after any number of cached ones; all keys
//   are read from the pages, so the step's own must be stored first.  Grid (query tiles of 32,
//   virtual heads, sequences), 128 threads: thread t works on query row t / 4; its 4 threads split
//   the tile's 32 keys (scores) and the value's elements (output).  Key tiles wholly outside the
//   tile's windows are skipped.
// attn_window_decode: one query per sequence; a block takes up to four virtual heads of one kv
//   head and one map, and one of `splits` ranges of the window's keys; a warp 32 keys at a time (a
//   lane a key for the scores, then the lanes the value's elements); ranges are merged by a second
//   kernel when there are several (ti_attn_window_merge serves the tensor-core decode kernel of
//   attn_decode_mma.cu the same way, which takes bfloat16 single tokens where it can).
// diff_combine: o = a1 - lambda a2 of the two maps' outputs, o / rms(o) * (1 - diff) * sigmoid(gate).
#include "common.cuh"

#include <algorithm>
#include <type_traits>

namespace {

struct Pages {
    const void* k_pages; const void* v_pages;      // [pages, kv_heads, page_size, maps * dim] and [.., vdim]
    const int* page_table; int table_width; int page_size; int n_pages;
};

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T>
__global__ void attn_window_prepare_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ bias,
                                           const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                           const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, int max_pos,
                                           const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                           const int* __restrict__ seq_slot, Pages pg, int H, int G, int maps, int dim, int vdim) {
    ti_pdl_trigger();
    extern __shared__ float sm[];       // the row as floats, then 33 for the sums
    const int nq = H * maps * dim, nk = G * maps * dim, nv = G * vdim, N = nq + nk + nv;
    float* red = sm + N;
    // where the token's keys and values go does not depend on the kernel before this one: the step's positions, slots and
    // page table were uploaded before its first kernel
    const int m = blockIdx.x;
    const int p = tok_pos[m], slot = seq_slot[tok_seq[m]];
    const int pidx = p / pg.page_size;
    const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : 0;
    ti_pdl_sync();
    qkv = ti_dependent(qkv);
    T* row = qkv + (size_t)m * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float x = to_f32(row[i]) + (bias ? bias[i] : 0.f);
        sm[i] = x;
        if (i < nq) sq = fmaf(x, x, sq);
        else if (i < nq + nk) sk = fmaf(x, x, sk);
    }
    float inv_q = 1.f, inv_k = 1.f;
    if (q_w) inv_q = rsqrtf(block_sum(sq, red) / (float)nq + eps);
    if (k_w) inv_k = rsqrtf(block_sum(sk, red) / (float)nk + eps);
    __syncthreads();
    const int pp = (page >= 0 && page < pg.n_pages) ? page : 0;       // page 0 is scratch
    const int prow = p % pg.page_size;
    const int half = rot >> 1, kw = maps * dim;
    const float* cs = cos_t ? cos_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        if (i < nq + nk) {
            const bool is_q = i < nq;
            const int seg = is_q ? 0 : nq, j = i - seg, e = j % dim;
            const float* w = is_q ? q_w : k_w;
            const float inv = is_q ? inv_q : inv_k;
            float x = sm[i];
            if (w) x = x * inv * w[j];
            if (cs && e < rot) {
                const int jo = e < half ? j + half : j - half;      // the other element of the pair
                float o = sm[seg + jo];
                if (w) o = o * inv * w[jo];
                x = e < half ? x * cs[e] - o * sn[e] : x * cs[e - half] + o * sn[e - half];
            }
            const T y = from_f32<T>(x);
            row[i] = y;         // keys and values go back too: the tensor-core kernel reads the step's own from the row
            if (!is_q) {
                const int g = j / kw;
                ((T*)pg.k_pages)[(((size_t)pp * G + g) * pg.page_size + prow) * kw + (j - g * kw)] = y;
            }
        } else {
            const int j = i - nq - nk, g = j / vdim;
            const T y = from_f32<T>(sm[i]);
            row[i] = y;
            ((T*)pg.v_pages)[(((size_t)pp * G + g) * pg.page_size + prow) * vdim + (j - g * vdim)] = y;
        }
    }
}

// Two sums over the block at once; every thread gets both.  `red` is shared memory for 66 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a); b = warp_sum(b);
    __syncthreads();        // protects `red` against a previous use
    if (lane == 0) { red[warp] = a; red[33 + warp] = b; }
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    if (warp == 0) {
        float ta = lane < nw ? red[lane] : 0.f, tb = lane < nw ? red[33 + lane] : 0.f;
        ta = warp_sum(ta); tb = warp_sum(tb);
        if (lane == 0) { red[32] = ta; red[65] = tb; }
    }
    __syncthreads();
    a = red[32]; b = red[65];
}

// E consecutive floats rounded to T and written by one 16-byte store (E * sizeof(T) == 16)
template <typename T, int E>
__device__ __forceinline__ void store_run16(T* __restrict__ p, const float (&x)[E]) {
    static_assert(E * sizeof(T) == 16, "one 16-byte store");
    T raw[E];
#pragma unroll
    for (int e = 0; e < E; e++) raw[e] = from_f32<T>(x[e]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(raw);
}

// The same work on runs of 16 bytes: every size that decides where a run lies (dim, vdim, the row stride) is a multiple of
// a run's E elements and every pointer is 16-byte aligned, so a run stays within one head and one map.
template <typename T>
__global__ void attn_window_prepare_vec_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ bias,
                                               const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, int max_pos,
                                               const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                               const int* __restrict__ seq_slot, Pages pg, int H, int G, int maps, int dim, int vdim) {
    ti_pdl_trigger();
    constexpr int E = 16 / (int)sizeof(T);
    extern __shared__ __align__(16) float sm[];       // the row as floats, then 66 for the sums
    const int nq = H * maps * dim, nk = G * maps * dim, nv = G * vdim, N = nq + nk + nv;
    float* red = sm + N;
    const int m = blockIdx.x;
    const int p = tok_pos[m], slot = seq_slot[tok_seq[m]];
    const int pidx = p / pg.page_size;
    const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : 0;
    ti_pdl_sync();
    qkv = ti_dependent(qkv);
    T* row = qkv + (size_t)m * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x * E; i < N; i += blockDim.x * E) {
        float x[E];
        T raw[E];
        *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(row + i);
#pragma unroll
        for (int e = 0; e < E; e++) x[e] = to_f32(raw[e]);
        if (bias) {
#pragma unroll
            for (int e = 0; e < E; e += 4) {
                const float4 b4 = *reinterpret_cast<const float4*>(bias + i + e);
                x[e] += b4.x; x[e + 1] += b4.y; x[e + 2] += b4.z; x[e + 3] += b4.w;
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; e += 4) {
            *reinterpret_cast<float4*>(sm + i + e) = make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
            ss += x[e] * x[e] + x[e + 1] * x[e + 1] + x[e + 2] * x[e + 2] + x[e + 3] * x[e + 3];
        }
        if (i < nq) sq += ss;
        else if (i < nq + nk) sk += ss;
    }
    block_sum2(sq, sk, red);        // (its last barrier also makes the whole row visible)
    const float inv_q = q_w ? rsqrtf(sq / (float)nq + eps) : 1.f, inv_k = k_w ? rsqrtf(sk / (float)nk + eps) : 1.f;
    const int pp = (page >= 0 && page < pg.n_pages) ? page : 0;       // page 0 is scratch
    const int prow = p % pg.page_size;
    const int half = rot >> 1, kw = maps * dim;
    const float* cs = cos_t ? cos_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    for (int i = threadIdx.x * E; i < N; i += blockDim.x * E) {
        float x[E];
#pragma unroll
        for (int e = 0; e < E; e += 4) {
            const float4 v4 = *reinterpret_cast<const float4*>(sm + i + e);
            x[e] = v4.x; x[e + 1] = v4.y; x[e + 2] = v4.z; x[e + 3] = v4.w;
        }
        if (i < nq + nk) {
            const bool is_q = i < nq;
            const int seg = is_q ? 0 : nq, j = i - seg, e0 = j % dim;
            const float* w = is_q ? q_w : k_w;
            const float inv = is_q ? inv_q : inv_k;
            if (w) {
#pragma unroll
                for (int e = 0; e < E; e++) x[e] = x[e] * inv * w[j + e];
            }
            if (cs && e0 < rot) {
#pragma unroll
                for (int e = 0; e < E; e++) {
                    const int el = e0 + e;
                    if (el < rot) {
                        const int jo = el < half ? j + e + half : j + e - half;      // the other element of the pair
                        float o = sm[seg + jo];
                        if (w) o = o * inv * w[jo];
                        x[e] = el < half ? x[e] * cs[el] - o * sn[el] : x[e] * cs[el - half] + o * sn[el - half];
                    }
                }
            }
            store_run16<T, E>(row + i, x);      // keys and values go back too: the tensor-core kernel reads the step's own from the row
            if (!is_q) {
                const int g = j / kw;
                store_run16<T, E>((T*)pg.k_pages + (((size_t)pp * G + g) * pg.page_size + prow) * kw + (j - g * kw), x);
            }
        } else {
            const int j = i - nq - nk, g = j / vdim;
            store_run16<T, E>(row + i, x);
            store_run16<T, E>((T*)pg.v_pages + (((size_t)pp * G + g) * pg.page_size + prow) * vdim + (j - g * vdim), x);
        }
    }
}

// A warp per (token, head): the heads of a token's row are its n_heads queries, then n_kv_heads keys, then n_kv_heads values.
// Shared memory: a head's elements per warp.  pairing 0: element e < rot/2 turns with e + rot/2; 1: element 2e with 2e + 1.
template <typename T>
__global__ void attn_head_prepare_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ bias,
                                         const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, int pairing,
                                         int max_pos, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                         const int* __restrict__ seq_slot, Pages pg, long long rows, int H, int G, int dim, int vdim,
                                         int width) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= rows) return;                                  // (warps never meet at a block-wide barrier)
    float* x = sm + (size_t)warp * width;
    const int per = H + 2 * G;
    const long long m = r / per;
    const int j = (int)(r - m * per);
    const int kind = j < H ? 0 : j < H + G ? 1 : 2;         // query, key, value
    const int head = kind == 0 ? j : kind == 1 ? j - H : j - H - G;
    const int n = kind == 2 ? vdim : dim;
    const int off = kind == 0 ? head * dim : kind == 1 ? H * dim + head * dim : (H + G) * dim + head * vdim;
    // where the token's keys and values go does not depend on the kernel before this one
    const int p = tok_pos[m], slot = seq_slot[tok_seq[m]];
    const int pidx = p / pg.page_size;
    const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : 0;
    ti_pdl_sync();
    qkv = ti_dependent(qkv);
    T* row = qkv + (size_t)m * ld + off;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float v = to_f32(row[i]) + (bias ? bias[off + i] : 0.f);
        x[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float* w = kind == 0 ? q_w : kind == 1 ? k_w : nullptr;
    if (w) {
        const float inv = rsqrtf(warp_sum(ss) / (float)n + eps);
        for (int i = lane; i < n; i += 32) x[i] = x[i] * inv * w[i];
    }
    __syncwarp();
    const int pp = (page >= 0 && page < pg.n_pages) ? page : 0;       // page 0 is scratch
    const size_t at = ((size_t)pp * G + head) * pg.page_size + p % pg.page_size;
    T* cache = kind == 1 ? (T*)pg.k_pages + at * dim : kind == 2 ? (T*)pg.v_pages + at * vdim : nullptr;
    const bool turns = cos_t && kind != 2;
    const int half = rot >> 1;
    const float* cs = cos_t ? cos_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    for (int i = lane; i < n; i += 32) {
        float v = x[i];
        if (turns && i < rot) {
            const bool first = pairing ? !(i & 1) : i < half;
            const int e = pairing ? i >> 1 : (first ? i : i - half);
            const float o = x[pairing ? i ^ 1 : (first ? i + half : i - half)];
            v = first ? v * cs[e] - o * sn[e] : v * cs[e] + o * sn[e];
        }
        const T y = from_f32<T>(v);
        row[i] = y;
        if (cache) cache[i] = y;
    }
}

constexpr int BQ = 32, BKV = 32, THREADS = 128;

template <typename T, typename OT, int MAXC, int MODE>
__global__ void __launch_bounds__(THREADS)
attn_window_kernel(const T* __restrict__ q, long long q_stride, OT* __restrict__ out, long long o_stride,
                   const int* __restrict__ cu_new, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                   Pages pg, const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ pb,
                   int n_heads, int n_kv_heads, int maps, int dim, int vdim, float scale, int window, int keep_first,
                   float out_scale) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    q = ti_dependent(q);
    const int ldk = dim + 1, ldv = vdim + 1;
    float* Qs = sm;                      // [BQ][dim + 1]
    float* Ks = Qs + BQ * ldk;           // [BKV][dim + 1]
    float* Vs = Ks + BKV * ldk;          // [BKV][vdim + 1]
    float* Ps = Vs + BKV * ldv;          // [BQ][BKV + 1]
    const int b = blockIdx.z, hv = blockIdx.y, q0 = blockIdx.x * BQ;
    const int tok0 = cu_new[b];
    const int n = cu_new[b + 1] - tok0;
    if (q0 >= n) return;
    const int h = hv / maps, map = hv - h * maps;
    const int kvh = h / (n_heads / n_kv_heads);
    const int kw = maps * dim, koff = map * dim;
    const int t = threadIdx.x, r = t >> 2, c4 = t & 3;
    const int start = seq_start[b], slot = seq_slot[b];
    const int end = start + n;
    const float a1 = r1 ? r1[h] : 0.f, a2 = r2 ? r2[h] : 0.f, hb = pb ? pb[h] : 0.f;

    for (int idx = t; idx < BQ * dim; idx += THREADS) {
        const int rr = idx / dim, d = idx - rr * dim;
        Qs[rr * ldk + d] = (q0 + rr < n) ? to_f32(q[(size_t)(tok0 + q0 + rr) * q_stride + (size_t)hv * dim + d]) : 0.f;
    }
    float acc[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; c++) acc[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int qi = start + q0 + r;      // this thread's query position
    const int nc = (vdim + 3) >> 2;     // value elements per thread (c4, c4 + 4, ...)
    const int last_q = start + min(q0 + BQ, n) - 1;
    const int first_k = window > 0 ? max(0, start + q0 - (window - 1)) : 0;
    // key tiles: those of the kept first positions that lie before the window's first tile, then the window's own
    const int k_band = (first_k / BKV) * BKV;
    const int keep_tiles = (min(keep_first, k_band) + BKV - 1) / BKV;
    const int n_tiles = keep_tiles + (last_q - k_band) / BKV + 1;
    for (int it = 0; it < n_tiles; it++) {
        const int k0 = it < keep_tiles ? it * BKV : k_band + (it - keep_tiles) * BKV;
        __syncthreads();  // previous tile fully consumed (and Qs written, first time)
        for (int rr = t >> 3; rr < BKV; rr += THREADS >> 3) {
            const int p = k0 + rr;
            const T* kp = nullptr;
            const T* vp = nullptr;
            if (p < end) {
                const int pidx = p / pg.page_size;
                const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : -1;
                if (page >= 0 && page < pg.n_pages) {
                    const size_t at = ((size_t)page * n_kv_heads + kvh) * pg.page_size + p % pg.page_size;
                    kp = (const T*)pg.k_pages + at * kw + koff;
                    vp = (const T*)pg.v_pages + at * vdim;
                }
            }
            for (int d = t & 7; d < dim; d += 8) Ks[rr * ldk + d] = kp ? to_f32(kp[d]) : 0.f;
            for (int d = t & 7; d < vdim; d += 8) Vs[rr * ldv + d] = vp ? to_f32(vp[d]) : 0.f;
        }
        __syncthreads();
        float s[8];
#pragma unroll
        for (int c = 0; c < 8; c++) s[c] = 0.f;
        const float* qrow = Qs + r * ldk;
        for (int d = 0; d < dim; d++) {
            const float qv = qrow[d];
#pragma unroll
            for (int c = 0; c < 8; c++) s[c] = fmaf(qv, Ks[(c4 + 4 * c) * ldk + d], s[c]);
        }
        bool okc[8];
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int kj = k0 + c4 + 4 * c;
            okc[c] = kj <= qi && kj < end && (window <= 0 || qi - kj < window || kj < keep_first);
            float x = s[c] * scale;
            if (r1 && okc[c]) x -= a1 * log1pf(a2 * (float)(qi - kj));
            s[c] = x;
        }
        if constexpr (MODE == 1) {
#pragma unroll
            for (int c = 0; c < 8; c++) Ps[r * (BKV + 1) + c4 + 4 * c] = okc[c] ? sigmoidf(s[c] + hb) : 0.f;
        } else {
            float m_tile = -INFINITY;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                s[c] = okc[c] ? s[c] : -INFINITY;
                m_tile = fmaxf(m_tile, s[c]);
            }
            m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
            m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
            const float m_new = fmaxf(m_run, m_tile);
            float alpha = 1.f, l_tile = 0.f;
            if (m_new > -INFINITY) {
                alpha = expf(m_run - m_new);  // exp(-inf) = 0 on the first useful tile
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const float p = expf(s[c] - m_new);
                    Ps[r * (BKV + 1) + c4 + 4 * c] = p;
                    l_tile += p;
                }
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) Ps[r * (BKV + 1) + c4 + 4 * c] = 0.f;
            }
            l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 1);
            l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 2);
            l_run = l_run * alpha + l_tile;
            m_run = m_new;
#pragma unroll
            for (int c = 0; c < MAXC; c++) acc[c] *= alpha;
        }
        __syncwarp();  // the four threads of a row are in one warp
        const float* prow = Ps + r * (BKV + 1);
        for (int j = 0; j < BKV; j++) {
            const float p = prow[j];
            const float* vrow = Vs + j * ldv + c4;
#pragma unroll
            for (int c = 0; c < MAXC; c++)
                if (c < nc && c4 + 4 * c < vdim) acc[c] = fmaf(p, vrow[4 * c], acc[c]);
        }
    }
    if (qi < end) {
        float inv = out_scale;
        if constexpr (MODE == 0) inv = l_run > 0.f ? out_scale / l_run : 0.f;
        OT* orow = out + (size_t)(tok0 + qi - start) * o_stride + (size_t)hv * vdim;
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc && c4 + 4 * c < vdim) orow[c4 + 4 * c] = from_f32<OT>(acc[c] * inv);
    }
}

constexpr int DEC_WARPS = 4, DEC_MAXE = 8;      // up to 256 elements per head, lane + 32 e

// `n` consecutive elements of a row as floats, by one load where size and address allow it
template <typename T, int N>
__device__ __forceinline__ void load_run(const T* __restrict__ p, float (&x)[N], bool vec) {
    constexpr int BYTES = N * (int)sizeof(T);
    if (vec && (BYTES == 16 || BYTES == 8 || BYTES == 4)) {
        T raw[N];
        if constexpr (BYTES == 16) *reinterpret_cast<uint4*>(raw) = *reinterpret_cast<const uint4*>(p);
        else if constexpr (BYTES == 8) *reinterpret_cast<uint2*>(raw) = *reinterpret_cast<const uint2*>(p);
        else if constexpr (BYTES == 4) *reinterpret_cast<uint32_t*>(raw) = *reinterpret_cast<const uint32_t*>(p);
#pragma unroll
        for (int e = 0; e < N; e++) x[e] = to_f32(raw[e]);
    } else {
#pragma unroll
        for (int e = 0; e < N; e++) x[e] = to_f32(p[e]);
    }
}

// The same for bfloat16 heads of 64, 128 or 256 elements on 16-byte-aligned rows: a lane holds 8 neighbouring elements of
// a head in registers (one 16-byte load, one 16-byte store to the row and one to the cache), LANES = max(dim, vdim) / 8
// lanes stand for a head (those past a shorter head's end idle) and a warp works on 32 / LANES heads at once; the sum of
// squares is a shuffle among a head's lanes, a neighbour pair lies within a lane and a half pair rot / 16 lanes further on.
template <int LANES>
__global__ void attn_head_prepare_vec_kernel(bf16* __restrict__ qkv, long long ld, const float* __restrict__ bias,
                                             const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                             const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, int pairing,
                                             int max_pos, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                             const int* __restrict__ seq_slot, Pages pg, long long rows, int H, int G, int dim, int vdim) {
    ti_pdl_trigger();
    constexpr int E = 8, RPW = 32 / LANES;
    const int lane = threadIdx.x & 31, l = lane % LANES;
    const long long r = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + lane / LANES;
    const bool live = r < rows;
    const int per = H + 2 * G;
    const long long m = live ? r / per : 0;
    const int j = live ? (int)(r - m * per) : 0;
    const int kind = j < H ? 0 : j < H + G ? 1 : 2;         // query, key, value
    const int head = kind == 0 ? j : kind == 1 ? j - H : j - H - G;
    const int n = kind == 2 ? vdim : dim;
    const int off = kind == 0 ? head * dim : kind == 1 ? H * dim + head * dim : (H + G) * dim + head * vdim;
    const int i0 = l * E;
    const bool mine = live && i0 < n;
    // where the token's keys and values go does not depend on the kernel before this one
    const int p = tok_pos[m], slot = seq_slot[tok_seq[m]];
    const int pidx = p / pg.page_size;
    const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : 0;
    const int pp = (page >= 0 && page < pg.n_pages) ? page : 0;       // page 0 is scratch
    const size_t at = ((size_t)pp * G + head) * pg.page_size + p % pg.page_size;
    bf16* cache = kind == 1 ? (bf16*)pg.k_pages + at * dim : kind == 2 ? (bf16*)pg.v_pages + at * vdim : nullptr;
    const bool turns = cos_t && kind != 2;
    const int half = rot >> 1;
    const float* cs = turns ? cos_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    const float* sn = turns ? sin_t + (size_t)min(p, max_pos - 1) * half : nullptr;
    const float* w = kind == 0 ? q_w : kind == 1 ? k_w : nullptr;
    ti_pdl_sync();
    qkv = ti_dependent(qkv);
    bf16* row = qkv + (size_t)m * ld + off;
    float x[E];
#pragma unroll
    for (int e = 0; e < E; e++) x[e] = 0.f;
    if (mine) load_run<bf16, E>(row + i0, x, true);
    float ss = 0.f;
    if (mine) {
        if (bias) {
            const float4 b0 = *reinterpret_cast<const float4*>(bias + off + i0), b1 = *reinterpret_cast<const float4*>(bias + off + i0 + 4);
            x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w; x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
        }
#pragma unroll
        for (int e = 0; e < E; e++) ss = fmaf(x[e], x[e], ss);
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);      // among a head's lanes
    if (mine && w) {
        const float inv = rsqrtf(ss / (float)n + eps);
#pragma unroll
        for (int e = 0; e < E; e++) x[e] = x[e] * inv * w[i0 + e];
    }
    if (cos_t) {                // (the same for the whole grid: every lane takes part in the exchange)
        if (pairing) {
            if (mine && turns) {
#pragma unroll
                for (int e = 0; e < E; e += 2) {
                    if (i0 + e < rot) {
                        const float c = cs[(i0 + e) >> 1], sv = sn[(i0 + e) >> 1], a = x[e], b = x[e + 1];
                        x[e] = a * c - b * sv;
                        x[e + 1] = b * c + a * sv;
                    }
                }
            }
        } else {
            const int hop = half / E;                   // lanes between the two elements of a pair (rot / 2 is a multiple of 8)
            const bool first = i0 < half;
#pragma unroll
            for (int e = 0; e < E; e++) {
                const float o = __shfl_sync(0xffffffffu, x[e], first ? lane + hop : lane - hop);      // (lanes outside the rotation read anything)
                if (mine && turns && i0 < rot) {
                    const int f = first ? i0 + e : i0 + e - half;
                    x[e] = first ? x[e] * cs[f] - o * sn[f] : x[e] * cs[f] + o * sn[f];
                }
            }
        }
    }
    if (mine) {
        store_run16<bf16, E>(row + i0, x);
        if (cache) store_run16<bf16, E>(cache + i0, x);
    }
}

// A block takes GH virtual heads of one kv head and one map, and one range of the window's keys.
// part_o [n_seq, virtual heads, splits, vdim], part_ml [n_seq, virtual heads, splits, 2] when splits > 1.
template <typename T, typename OT, int GH, int VPL, int MODE>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_window_decode_kernel(const T* __restrict__ q, long long q_stride, OT* __restrict__ out, long long o_stride,
                          const int* __restrict__ seq_len, const int* __restrict__ seq_slot, Pages pg,
                          const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ pb,
                          int n_heads, int n_kv_heads, int maps, int dim, int vdim, float scale, int window, int keep_first,
                          float out_scale, int splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    ti_pdl_trigger();
    extern __shared__ __align__(16) float dsm[];         // q: [GH][dim]; o: [DEC_WARPS][GH][32 * VPL]; m, l: [DEC_WARPS][GH][2]
    float* q_sh = dsm;
    float* o_sh = q_sh + GH * dim;
    float* ml_sh = o_sh + DEC_WARPS * GH * 32 * VPL;
    ti_pdl_sync();
    q = ti_dependent(q);
    const int b = blockIdx.z, sp = blockIdx.x;
    const int group = n_heads / n_kv_heads, cpg = group / GH;        // chunks of GH heads per kv head and map
    const int kvh = blockIdx.y / (maps * cpg), rem = blockIdx.y - kvh * maps * cpg;
    const int map = rem / cpg, h0 = kvh * group + (rem - map * cpg) * GH;
    const int kw = maps * dim, koff = map * dim;
    const int len = seq_len[b], slot = seq_slot[b];
    const int qi = len - 1;
    const int lo = window > 0 ? max(0, len - window) : 0;           // first visible key
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t_first = lo / 32, tiles = (len + 31) / 32;
    // tiles of 32 keys in the order they are shared out: those of the kept first positions that lie before the window's
    // first tile, then the window's own
    const int keep_tiles = min((keep_first + 31) / 32, t_first);
    const int n_tiles = keep_tiles + tiles - t_first;
    const int per = (n_tiles + splits - 1) / splits;
    const int t_lo = sp * per, t_hi = min(n_tiles, t_lo + per);
    for (int i = threadIdx.x; i < GH * dim; i += DEC_WARPS * 32) {
        const int g = i / dim, d = i - g * dim;
        q_sh[i] = to_f32(q[(size_t)b * q_stride + (size_t)((h0 + g) * maps + map) * dim + d]) * scale;
    }
    __syncthreads();
    const bool kvec = (dim * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(pg.k_pages) & 15) == 0;
    const bool vvec = vdim % VPL == 0 && (reinterpret_cast<uintptr_t>(pg.v_pages) & 15) == 0;
    constexpr int KPER = 16 / sizeof(T);
    float acc[GH][VPL], m_run[GH], l_run[GH], a1[GH], a2[GH], hb[GH];
#pragma unroll
    for (int g = 0; g < GH; g++) {
        m_run[g] = MODE == 1 ? 0.f : -INFINITY; l_run[g] = 0.f;
        a1[g] = r1 ? r1[h0 + g] : 0.f; a2[g] = r2 ? r2[h0 + g] : 0.f; hb[g] = pb ? pb[h0 + g] : 0.f;
#pragma unroll
        for (int e = 0; e < VPL; e++) acc[g][e] = 0.f;
    }
    for (int vt = t_lo + warp; vt < t_hi; vt += DEC_WARPS) {
        const int t = vt < keep_tiles ? vt : t_first + vt - keep_tiles;
        const int j = t * 32 + lane;
        int at = -1;                                     // the key's row among all rows of the pages
        if (j < len && (j >= lo || j < keep_first)) {
            const int pidx = j / pg.page_size;
            const int page = pidx < pg.table_width ? pg.page_table[(size_t)slot * pg.table_width + pidx] : -1;
            if (page >= 0 && page < pg.n_pages) at = (page * n_kv_heads + kvh) * pg.page_size + j % pg.page_size;
        }
        float s[GH];
#pragma unroll
        for (int g = 0; g < GH; g++) s[g] = 0.f;
        if (at >= 0) {
            const T* kp = (const T*)pg.k_pages + (size_t)at * kw + koff;
            if (kvec) {
                for (int d = 0; d < dim; d += KPER) {
                    float x[KPER];
                    load_run<T, KPER>(kp + d, x, true);
#pragma unroll
                    for (int g = 0; g < GH; g++)
#pragma unroll
                        for (int e = 0; e < KPER; e++) s[g] = fmaf(q_sh[g * dim + d + e], x[e], s[g]);
                }
            } else {
                for (int d = 0; d < dim; d++) {
                    const float x = to_f32(kp[d]);
#pragma unroll
                    for (int g = 0; g < GH; g++) s[g] = fmaf(q_sh[g * dim + d], x, s[g]);
                }
            }
        }
        float p[GH];
        bool any = false;
#pragma unroll
        for (int g = 0; g < GH; g++) {
            float x = s[g];
            if (r1 && at >= 0) x -= a1[g] * log1pf(a2[g] * (float)(qi - j));
            if constexpr (MODE == 1) {
                p[g] = at >= 0 ? sigmoidf(x + hb[g]) : 0.f;
                any = true;
            } else {
                x = at >= 0 ? x : -INFINITY;
                const float m_new = fmaxf(m_run[g], warp_max(x));
                p[g] = 0.f;
                if (m_new > -INFINITY) {                     // (the same for all lanes)
                    const float alpha = expf(m_run[g] - m_new);
                    p[g] = at >= 0 ? expf(x - m_new) : 0.f;
                    l_run[g] = l_run[g] * alpha + warp_sum(p[g]);
                    m_run[g] = m_new;
#pragma unroll
                    for (int e = 0; e < VPL; e++) acc[g][e] *= alpha;
                    any = true;
                }
            }
        }
        if (!any) continue;
#pragma unroll 4
        for (int jj = 0; jj < 32; jj++) {
            const int aj = __shfl_sync(0xffffffffu, at, jj);
            float x[VPL];
#pragma unroll
            for (int e = 0; e < VPL; e++) x[e] = 0.f;
            const T* vp = (const T*)pg.v_pages + (size_t)max(aj, 0) * vdim + lane * VPL;
            if (vvec) {
                if (lane * VPL < vdim) load_run<T, VPL>(vp, x, true);
            } else {
#pragma unroll
                for (int e = 0; e < VPL; e++) x[e] = lane * VPL + e < vdim ? to_f32(vp[e]) : 0.f;
            }
#pragma unroll
            for (int g = 0; g < GH; g++) {
                const float pj = __shfl_sync(0xffffffffu, p[g], jj);       // 0 where the lane's key does not exist
#pragma unroll
                for (int e = 0; e < VPL; e++)
                    if (aj >= 0 && lane * VPL + e < vdim) acc[g][e] = fmaf(pj, x[e], acc[g][e]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GH; g++) {
#pragma unroll
        for (int e = 0; e < VPL; e++) o_sh[(warp * GH + g) * 32 * VPL + lane * VPL + e] = acc[g][e];
        if (lane == 0) { ml_sh[(warp * GH + g) * 2] = m_run[g]; ml_sh[(warp * GH + g) * 2 + 1] = l_run[g]; }
    }
    __syncthreads();
    for (int g = 0; g < GH; g++) {
        const int hv = (h0 + g) * maps + map;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; w++) m_all = fmaxf(m_all, ml_sh[(w * GH + g) * 2]);
        float l_all = 0.f, f[DEC_WARPS];
#pragma unroll
        for (int w = 0; w < DEC_WARPS; w++) {
            const float mw = ml_sh[(w * GH + g) * 2];
            f[w] = mw > -INFINITY ? expf(mw - m_all) : 0.f;          // MODE 1: every m is 0 and every f is 1
            l_all += ml_sh[(w * GH + g) * 2 + 1] * f[w];
        }
        for (int d = threadIdx.x; d < vdim; d += DEC_WARPS * 32) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; w++) o = fmaf(o_sh[(w * GH + g) * 32 * VPL + d], f[w], o);
            if (splits == 1) {
                if constexpr (MODE == 0) o = l_all > 0.f ? o / l_all : 0.f;
                out[(size_t)b * o_stride + (size_t)hv * vdim + d] = from_f32<OT>(o * out_scale);
            } else {
                part_o[(((size_t)b * n_heads * maps + hv) * splits + sp) * vdim + d] = o;
            }
        }
        if (splits > 1 && threadIdx.x == 0) {
            float* ml = part_ml + (((size_t)b * n_heads * maps + hv) * splits + sp) * 2;
            ml[0] = m_all; ml[1] = l_all;
        }
    }
}

template <typename OT, int MODE>
__global__ void attn_window_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, OT* __restrict__ out,
                                         long long o_stride, int n_virtual, int vdim, int splits, float out_scale) {
    ti_pdl_trigger();
    ti_pdl_sync();
    part_o = ti_dependent(part_o); part_ml = ti_dependent(part_ml);
    const int b = blockIdx.y, hv = blockIdx.x;
    const float* ml = part_ml + ((size_t)b * n_virtual + hv) * splits * 2;
    const float* po = part_o + ((size_t)b * n_virtual + hv) * splits * vdim;
    if constexpr (MODE == 1) {
        for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
            float o = 0.f;
            for (int s = 0; s < splits; s++) o += po[(size_t)s * vdim + d];
            out[(size_t)b * o_stride + (size_t)hv * vdim + d] = from_f32<OT>(o * out_scale);
        }
        return;
    }
    float m_all = -INFINITY;
    for (int s = 0; s < splits; s++) m_all = fmaxf(m_all, ml[2 * s]);
    float l_all = 0.f;
    for (int s = 0; s < splits; s++) l_all += ml[2 * s] > -INFINITY ? ml[2 * s + 1] * expf(ml[2 * s] - m_all) : 0.f;
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; s++)
            if (ml[2 * s] > -INFINITY) o = fmaf(po[(size_t)s * vdim + d], expf(ml[2 * s] - m_all), o);
        out[(size_t)b * o_stride + (size_t)hv * vdim + d] = from_f32<OT>(l_all > 0.f ? o / l_all * out_scale : 0.f);
    }
}

// a warp per (token, head)
template <typename T>
__global__ void diff_combine_kernel(const float* __restrict__ a, const T* __restrict__ gate, long long g_stride, T* __restrict__ out,
                                    long long o_stride, int M, int H, int vdim, float lambda, float diff, float eps) {
    ti_pdl_trigger();
    ti_pdl_sync();
    a = ti_dependent(a); gate = ti_dependent(gate);
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= (long long)M * H) return;
    const int lane = threadIdx.x & 31;
    const int m = (int)(r / H), h = (int)(r - (long long)m * H);
    const float* a1 = a + (size_t)r * 2 * vdim;
    const float* a2 = a1 + vdim;
    float ss = 0.f;
    for (int e = lane; e < vdim; e += 32) {
        const float o = a1[e] - lambda * a2[e];
        ss = fmaf(o, o, ss);
    }
    float f = rsqrtf(warp_sum(ss) / (float)vdim + eps) * (1.0f - diff);
    if (gate) f *= sigmoidf(to_f32(gate[(size_t)m * g_stride + h]));
    for (int e = lane; e < vdim; e += 32)
        out[(size_t)m * o_stride + (size_t)h * vdim + e] = from_f32<T>((a1[e] - lambda * a2[e]) * f);
}

int check_pages(const char* what, const void* k_pages, const void* v_pages, const int* page_table, int table_width, int page_size,
                int n_pages) {
    TI_REQUIRE(k_pages && v_pages && page_table && page_size > 0 && table_width > 0 && n_pages > 0, "%s: incomplete cache description", what);
    return 0;
}

}  // namespace

// qkv: [M, >= heads * maps * dim + kv_heads * (maps * dim + vdim)] of the engine's type, row stride ld (columns after q, k, v
// are left alone); bias: float32 of q, k and v's length or null; q_w: float32 [heads * maps * dim] or null; k_w: float32
// [kv_heads * maps * dim] or null; cos_t, sin_t: float32 [max_pos, rot / 2] or null.
extern "C" int ti_attn_window_prepare(void* qkv, long long ld, const float* bias, const float* q_w, const float* k_w, float eps,
                                      const float* cos_t, const float* sin_t, int rot, int max_pos, const int* tok_pos,
                                      const int* tok_seq, const int* seq_slot, void* k_pages, void* v_pages, const int* page_table,
                                      int table_width, int page_size, int n_pages, int M, int n_heads, int n_kv_heads, int maps,
                                      int dim, int vdim, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && n_kv_heads > 0 && maps > 0 && dim > 0 && vdim > 0, "attn_window_prepare: bad sizes");
    TI_REQUIRE(!cos_t || (sin_t && rot > 0 && rot % 2 == 0 && rot <= dim && max_pos > 0),
               "attn_window_prepare: a rotation of %d of %d elements with tables of %d positions", rot, dim, max_pos);
    if (check_pages("attn_window_prepare", k_pages, v_pages, page_table, table_width, page_size, n_pages)) return 1;
    Pages pg{k_pages, v_pages, page_table, table_width, page_size, n_pages};
    const long long N = (long long)n_heads * maps * dim + (long long)n_kv_heads * (maps * dim + vdim);
    const size_t smem = (size_t)(N + 66) * sizeof(float);
    TI_REQUIRE(smem <= 200 * 1024, "attn_window_prepare: a projection row of %lld elements does not fit shared memory", N);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        static size_t configured = 0;
        if (smem > 48 * 1024 && smem > configured) {
            TI_CUDA(cudaFuncSetAttribute(attn_window_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured = smem;
        }
        constexpr int E = 16 / (int)sizeof(T);
        auto a16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
        if (dim % E == 0 && vdim % E == 0 && ld % E == 0 && a16(qkv) && a16(bias) && a16(q_w) && a16(k_w) && a16(k_pages) && a16(v_pages)) {
            static size_t configured_vec = 0;
            if (smem > 48 * 1024 && smem > configured_vec) {
                TI_CUDA(cudaFuncSetAttribute(attn_window_prepare_vec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured_vec = smem;
            }
            // a run a thread when the tokens are few (the step is a chain of latencies), two when they fill the device
            // several times over (more blocks at once)
            const long long runs = (N / E + (M >= 592 ? 1 : 0)) / (M >= 592 ? 2 : 1);
            TI_CUDA(ti_launch_class<2>(attn_window_prepare_vec_kernel<T>, dim3(M), dim3((unsigned)std::min<long long>(512, (runs + 31) / 32 * 32)), smem, stream,
                                       (T*)qkv, ld, bias, q_w, k_w, eps, cos_t, sin_t, cos_t ? rot : 0, max_pos, tok_pos, tok_seq, seq_slot, pg,
                                       n_heads, n_kv_heads, maps, dim, vdim));
            TI_CHECK_LAUNCH("attn_window_prepare (16-byte runs)");
            return 0;
        }
        TI_CUDA(ti_launch_class<2>(attn_window_prepare_kernel<T>, dim3(M), dim3(N <= 1024 ? 128 : N <= 2048 ? 256 : 512), smem, stream, (T*)qkv, ld, bias,
                                   q_w, k_w, eps, cos_t, sin_t, cos_t ? rot : 0, max_pos, tok_pos, tok_seq, seq_slot, pg, n_heads,
                                   n_kv_heads, maps, dim, vdim));
        TI_CHECK_LAUNCH("attn_window_prepare");
        return 0;
    });
}

// qkv: [M, >= heads * dim + kv_heads * (dim + vdim)] of the engine's type, row stride ld (columns after q, k, v are left
// alone); bias: float32 of q, k and v's length or null; q_w, k_w: float32 [dim] or null (one weight for all heads); cos_t,
// sin_t: float32 [max_pos, rot / 2] or null; pairing 0: elements (e, e + rot / 2) turn together, 1: (2e, 2e + 1).
extern "C" int ti_attn_head_prepare(void* qkv, long long ld, const float* bias, const float* q_w, const float* k_w, float eps,
                                    const float* cos_t, const float* sin_t, int rot, int pairing, int max_pos, const int* tok_pos,
                                    const int* tok_seq, const int* seq_slot, void* k_pages, void* v_pages, const int* page_table,
                                    int table_width, int page_size, int n_pages, int M, int n_heads, int n_kv_heads, int dim,
                                    int vdim, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && n_kv_heads > 0 && dim > 0 && vdim > 0, "attn_head_prepare: bad sizes");
    TI_REQUIRE(!cos_t || (sin_t && rot > 0 && rot % 2 == 0 && rot <= dim && max_pos > 0 && (pairing == 0 || pairing == 1)),
               "attn_head_prepare: a rotation of %d of %d elements with tables of %d positions", rot, dim, max_pos);
    if (check_pages("attn_head_prepare", k_pages, v_pages, page_table, table_width, page_size, n_pages)) return 1;
    Pages pg{k_pages, v_pages, page_table, table_width, page_size, n_pages};
    const int width = std::max(dim, vdim), warps = 4;
    const size_t smem = (size_t)warps * width * sizeof(float);
    TI_REQUIRE(smem <= 48 * 1024, "attn_head_prepare: heads of %d elements are not supported", width);
    const long long rows = (long long)M * (n_heads + 2 * n_kv_heads);
    auto lanes = [](int n) { return n == 64 || n == 128 || n == 256; };
    auto a16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (dtype == TI_BF16 && lanes(dim) && lanes(vdim) && ld % 8 == 0 && a16(qkv) && a16(k_pages) && a16(v_pages) && a16(bias) &&
        (!cos_t || pairing == 1 || (rot / 2) % 8 == 0)) {
        const int group = std::max(dim, vdim) / 8;          // lanes that stand for a head
        const long long warps = (rows + 32 / group - 1) / (32 / group);
        const dim3 grid((unsigned)((warps + 3) / 4)), block(128);
#define TI_HEAD_PREPARE(L) TI_CUDA(ti_launch_class<2>(attn_head_prepare_vec_kernel<L>, grid, block, 0, stream, (bf16*)qkv, ld, bias, q_w, k_w, eps, \
            cos_t, sin_t, cos_t ? rot : 0, pairing, max_pos, tok_pos, tok_seq, seq_slot, pg, rows, n_heads, n_kv_heads, dim, vdim))
        if (group == 8) TI_HEAD_PREPARE(8); else if (group == 16) TI_HEAD_PREPARE(16); else TI_HEAD_PREPARE(32);
#undef TI_HEAD_PREPARE
        TI_CHECK_LAUNCH("attn_head_prepare (a lane a run)");
        return 0;
    }
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<2>(attn_head_prepare_kernel<T>, dim3((unsigned)((rows + warps - 1) / warps)), dim3(warps * 32), smem, stream,
                                   (T*)qkv, ld, bias, q_w, k_w, eps, cos_t, sin_t, cos_t ? rot : 0, pairing, max_pos, tok_pos, tok_seq,
                                   seq_slot, pg, rows, n_heads, n_kv_heads, dim, vdim, width));
        TI_CHECK_LAUNCH("attn_head_prepare");
        return 0;
    });
}

// q: [M, heads * maps, dim] (row stride q_stride); out: [M, heads * maps, vdim] (row stride o_stride), float32 when
// out_f32 else the engine's type; r1, r2, pb: float32 [heads] or null; mode 0 softmax, 1 sigmoid; window <= 0: all keys.
extern "C" int ti_attn_window(const void* q, long long q_stride, void* out, long long o_stride, int out_f32, const int* cu_new,
                              const int* seq_start, const int* seq_slot, int n_seq, int max_new, const void* k_pages,
                              const void* v_pages, const int* page_table, int table_width, int page_size, int n_pages,
                              const float* r1, const float* r2, const float* pb, int n_heads, int n_kv_heads, int maps, int dim,
                              int vdim, float scale, int window, int keep_first, float out_scale, int mode, int dtype,
                              cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(n_seq > 0 && max_new > 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && maps > 0, "attn_window: bad sizes");
    TI_REQUIRE(dim >= 1 && dim <= 256 && vdim >= 1 && vdim <= 256, "attn_window: heads of %d and %d elements are not supported (up to 256)", dim, vdim);
    TI_REQUIRE(n_seq <= 65535 && n_heads * maps <= 65535, "attn_window: too many sequences or heads for one launch");
    TI_REQUIRE(mode == 0 || mode == 1, "attn_window: unknown mode %d", mode);
    TI_REQUIRE(keep_first >= 0, "attn_window: %d kept first positions", keep_first);
    TI_REQUIRE((r1 == nullptr) == (r2 == nullptr), "attn_window: the distance term needs both of its constants");
    if (check_pages("attn_window", k_pages, v_pages, page_table, table_width, page_size, n_pages)) return 1;
    Pages pg{k_pages, v_pages, page_table, table_width, page_size, n_pages};
    const size_t smem = ((size_t)(BQ + BKV) * (dim + 1) + (size_t)BKV * (vdim + 1) + (size_t)BQ * (BKV + 1)) * sizeof(float);
    dim3 grid((max_new + BQ - 1) / BQ, n_heads * maps, n_seq);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto ot, auto mc, auto md) -> int {
            using OT = decltype(ot);
            constexpr int MAXC = decltype(mc)::value, MODE = decltype(md)::value;
            static size_t configured = 0;
            if (smem > configured) {
                TI_CUDA(cudaFuncSetAttribute(attn_window_kernel<T, OT, MAXC, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured = smem;
            }
            TI_CUDA(ti_launch(attn_window_kernel<T, OT, MAXC, MODE>, grid, dim3(THREADS), smem, stream, (const T*)q, q_stride, (OT*)out,
                              o_stride, cu_new, seq_start, seq_slot, pg, r1, r2, pb, n_heads, n_kv_heads, maps, dim, vdim, scale, window,
                              window > 0 ? keep_first : 0, out_scale));
            TI_CHECK_LAUNCH("attn_window");
            return 0;
        };
        auto with_mode = [&](auto ot, auto mc) -> int {
            return mode == 1 ? go(ot, mc, std::integral_constant<int, 1>()) : go(ot, mc, std::integral_constant<int, 0>());
        };
        auto with_c = [&](auto ot) -> int {
            if (vdim <= 64) return with_mode(ot, std::integral_constant<int, 16>());
            if (vdim <= 128) return with_mode(ot, std::integral_constant<int, 32>());
            return with_mode(ot, std::integral_constant<int, 64>());
        };
        return out_f32 ? with_c(float()) : with_c(T());
    });
}

// One query per sequence (its last position, seq_len - 1).  part_o: float32 [n_seq, heads * maps, splits, vdim] and
// part_ml: float32 [n_seq, heads * maps, splits, 2], both only when splits > 1.
extern "C" int ti_attn_window_decode(const void* q, long long q_stride, void* out, long long o_stride, int out_f32,
                                     const int* seq_len, const int* seq_slot, int n_seq, const void* k_pages, const void* v_pages,
                                     const int* page_table, int table_width, int page_size, int n_pages, const float* r1,
                                     const float* r2, const float* pb, int n_heads, int n_kv_heads, int maps, int dim, int vdim,
                                     float scale, int window, int keep_first, float out_scale, int mode, int splits, float* part_o,
                                     float* part_ml, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0 && maps > 0 && splits >= 1, "attn_window_decode: bad sizes");
    TI_REQUIRE(dim >= 1 && dim <= 32 * DEC_MAXE && vdim >= 1 && vdim <= 32 * DEC_MAXE,
               "attn_window_decode: heads of %d and %d elements are not supported (up to %d)", dim, vdim, 32 * DEC_MAXE);
    TI_REQUIRE(n_seq <= 65535 && n_heads * maps <= 65535, "attn_window_decode: too many sequences or heads for one launch");
    TI_REQUIRE(splits == 1 || (part_o && part_ml), "attn_window_decode: split keys need scratch");
    TI_REQUIRE(mode == 0 || mode == 1, "attn_window_decode: unknown mode %d", mode);
    TI_REQUIRE(keep_first >= 0, "attn_window_decode: %d kept first positions", keep_first);
    TI_REQUIRE((r1 == nullptr) == (r2 == nullptr), "attn_window_decode: the distance term needs both of its constants");
    if (check_pages("attn_window_decode", k_pages, v_pages, page_table, table_width, page_size, n_pages)) return 1;
    Pages pg{k_pages, v_pages, page_table, table_width, page_size, n_pages};
    // heads of one kv head (and one map) per block: as many of 4, 2, 1 as divide the group; value elements per lane: 1, 2, 4 or 8
    const int group = n_heads / n_kv_heads;
    const int gh = group % 4 == 0 ? 4 : group % 2 == 0 ? 2 : 1;
    const int vpl = vdim <= 32 ? 1 : vdim <= 64 ? 2 : vdim <= 128 ? 4 : 8;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto ot, auto md, auto ghv, auto vplv) -> int {
            using OT = decltype(ot);
            constexpr int MODE = decltype(md)::value, GH = decltype(ghv)::value, VPL = decltype(vplv)::value;
            const size_t smem = ((size_t)GH * dim + (size_t)DEC_WARPS * GH * 32 * VPL + (size_t)DEC_WARPS * GH * 2) * sizeof(float);
            static size_t configured = 0;
            if (smem > 48 * 1024 && smem > configured) {
                TI_CUDA(cudaFuncSetAttribute(attn_window_decode_kernel<T, OT, GH, VPL, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                configured = smem;
            }
            TI_CUDA(ti_launch_class<3>(attn_window_decode_kernel<T, OT, GH, VPL, MODE>, dim3(splits, n_heads * maps / GH, n_seq),
                                       dim3(DEC_WARPS * 32), smem, stream, (const T*)q, q_stride, (OT*)out, o_stride, seq_len, seq_slot, pg,
                                       r1, r2, pb, n_heads, n_kv_heads, maps, dim, vdim, scale, window, window > 0 ? keep_first : 0, out_scale, splits,
                                       part_o, part_ml));
            TI_CHECK_LAUNCH("attn_window_decode");
            if (splits > 1) {
                TI_CUDA(ti_launch_class<4>(attn_window_merge_kernel<OT, MODE>, dim3(n_heads * maps, n_seq), dim3(64), 0, stream,
                                           (const float*)part_o, (const float*)part_ml, (OT*)out, o_stride, n_heads * maps, vdim, splits, out_scale));
                TI_CHECK_LAUNCH("attn_window_merge");
            }
            return 0;
        };
        auto with_vpl = [&](auto ot, auto md, auto ghv) -> int {
            switch (vpl) {
                case 1: return go(ot, md, ghv, std::integral_constant<int, 1>());
                case 2: return go(ot, md, ghv, std::integral_constant<int, 2>());
                case 4: return go(ot, md, ghv, std::integral_constant<int, 4>());
                default: return go(ot, md, ghv, std::integral_constant<int, 8>());
            }
        };
        auto with_gh = [&](auto ot, auto md) -> int {
            return gh == 4 ? with_vpl(ot, md, std::integral_constant<int, 4>()) : gh == 2 ? with_vpl(ot, md, std::integral_constant<int, 2>())
                                                                                        : with_vpl(ot, md, std::integral_constant<int, 1>());
        };
        auto with_mode = [&](auto ot) -> int {
            return mode == 1 ? with_gh(ot, std::integral_constant<int, 1>()) : with_gh(ot, std::integral_constant<int, 0>());
        };
        return out_f32 ? with_mode(float()) : with_mode(T());
    });
}

// The merge alone, for partial results that another kernel left (the tensor-core kernel for single tokens): part_o
// [n_seq, virtual heads, splits, vdim], part_ml [n_seq, virtual heads, splits, 2] -> out [n_seq, virtual heads * vdim].
extern "C" int ti_attn_window_merge(const float* part_o, const float* part_ml, void* out, long long o_stride, int out_f32, int n_seq,
                                    int n_virtual, int vdim, int splits, int mode, float out_scale, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_seq <= 65535 && n_virtual > 0 && vdim > 0 && splits >= 1 && part_o && part_ml, "attn_window_merge: bad sizes");
    TI_REQUIRE(mode == 0 || mode == 1, "attn_window_merge: unknown mode %d", mode);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        auto go = [&](auto ot, auto md) -> int {
            using OT = decltype(ot);
            TI_CUDA(ti_launch_class<4>(attn_window_merge_kernel<OT, decltype(md)::value>, dim3(n_virtual, n_seq), dim3(64), 0, stream, part_o,
                                       part_ml, (OT*)out, o_stride, n_virtual, vdim, splits, out_scale));
            TI_CHECK_LAUNCH("attn_window_merge");
            return 0;
        };
        auto with_mode = [&](auto ot) -> int {
            return mode == 1 ? go(ot, std::integral_constant<int, 1>()) : go(ot, std::integral_constant<int, 0>());
        };
        return out_f32 ? with_mode(float()) : with_mode(T());
    });
}

// a: float32 [M, heads, 2, vdim] (the two maps' outputs); gate: [M, heads] logits of the engine's type with row stride
// g_stride, or null; out: [M, heads * vdim] with row stride o_stride:  (a1 - lambda a2) / rms(.) * (1 - diff) * sigmoid(gate).
extern "C" int ti_diff_combine(const float* a, const void* gate, long long g_stride, void* out, long long o_stride, int M, int n_heads,
                               int vdim, float lambda, float diff, float eps, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && n_heads > 0 && vdim > 0, "diff_combine: bad sizes");
    const long long rows = (long long)M * n_heads;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(diff_combine_kernel<T>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream, a, (const T*)gate, g_stride,
                                   (T*)out, o_stride, M, n_heads, vdim, lambda, diff, eps));
        TI_CHECK_LAUNCH("diff_combine");
        return 0;
    });
}
