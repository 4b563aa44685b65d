// A float32 residual stream between sublayers that are normed on the way in AND on the way out.
//
// A layer of such a design does  h <- h + n_post(f(n_pre(h)))  per sublayer f, with
// n(v) = v * rsqrt(mean(v^2) + eps) * w.  The sublayer's output y (engine type) stays pending
// until the next reader of the stream: this kernel forms n_post(y), adds it to the float32 row of
// h without rounding, writes the row back, and norms the new row for the next sublayer, all in
// one pass (one block per row).  With `rows` it works on the gathered rows only and leaves h
// alone (the head's rows).  A norm weight is float32, one number (stride 0) or one per channel
// (stride 1).
#include "common.cuh"

namespace {

template <typename T>
__global__ void post_norm_add_norm_kernel(float* __restrict__ h, const T* __restrict__ y, const float* __restrict__ w_post,
                                          int post_stride, const int* __restrict__ rows, const float* __restrict__ w_pre,
                                          int pre_stride, T* __restrict__ out, int H, int M, float eps, int write_back) {
    ti_pdl_trigger();
    extern __shared__ float row[];      // H floats + 33
    float* red = row + H;
    ti_pdl_sync();
    h = ti_dependent(h); y = ti_dependent(y);
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    const bool ok = src >= 0 && src < M;
    if (!ok) src = 0;
    const size_t base = (size_t)src * H;
    float inv_y = 0.f;
    if (y) {
        // the stream's row comes in with the pending output, so that the sum below waits for no second read of memory
        float sy = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = to_f32(y[base + i]);
            row[i] = h[base + i];
            sy = fmaf(v, v, sy);
        }
        inv_y = rsqrtf(block_sum(sy, red) / (float)H + eps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = y ? row[i] : h[base + i];        // (a thread reads back what it wrote itself)
        if (y) x += to_f32(y[base + i]) * inv_y * w_post[(size_t)i * post_stride];
        if (!ok) x = 0.f;
        row[i] = x;
        if (write_back && y) h[base + i] = x;
        ss = fmaf(x, x, ss);
    }
    if (!out) return;
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t)r * H + i] = from_f32<T>(row[i] * inv * w_pre[(size_t)i * pre_stride]);
}

}  // namespace

// h: float32 [M, H].  y: [M, H] of the engine's type or null (nothing pending).  w_post / w_pre: float32, one number
// (stride 0) or H (stride 1).  rows: null (every row, R == M) or R row indices.  out: [R, H] of the engine's type or
// null (only the sum is wanted).  write_back: store the sum into h.
extern "C" int ti_post_norm_add_norm(float* h, const void* y, const float* w_post, int post_stride, const int* rows,
                                     const float* w_pre, int pre_stride, void* out, int R, int H, int M, float eps,
                                     int write_back, int dtype, cudaStream_t stream) {
    if (R == 0) return 0;
    TI_REQUIRE(R > 0 && H > 0 && M > 0, "post_norm_add_norm: bad sizes R=%d H=%d M=%d", R, H, M);
    TI_REQUIRE(rows || R == M, "post_norm_add_norm: without row indices every row is taken (R=%d, M=%d)", R, M);
    TI_REQUIRE(!(rows && write_back), "post_norm_add_norm: gathered rows are not written back");
    TI_REQUIRE(!y || w_post, "post_norm_add_norm: a pending output needs its norm weight");
    TI_REQUIRE(!out || w_pre, "post_norm_add_norm: normed rows need a norm weight");
    TI_REQUIRE((post_stride == 0 || post_stride == 1) && (pre_stride == 0 || pre_stride == 1), "post_norm_add_norm: weight strides are 0 or 1");
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    TI_REQUIRE(smem <= 200 * 1024, "post_norm_add_norm: rows of %d elements do not fit shared memory", H);
    int threads = 256;
    if (H <= 256) threads = 64;
    else if (H <= 1024) threads = 128;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        static size_t configured = 0;
        if (smem > 48 * 1024 && smem > configured) {
            TI_CUDA(cudaFuncSetAttribute(post_norm_add_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured = smem;
        }
        TI_CUDA(ti_launch_class<1>(post_norm_add_norm_kernel<T>, dim3(R), dim3(threads), smem, stream, h, (const T*)y, w_post,
                                   post_stride, rows, w_pre, pre_stride, (T*)out, H, M, eps, write_back));
        TI_CHECK_LAUNCH("post_norm_add_norm");
        return 0;
    });
}

namespace {

__device__ __forceinline__ float gate_act(float g, int act) {
    if (act == 1) {      // the tanh form of gelu
        const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.0f + tanhf(u));
    }
    return g / (1.0f + expf(-g));       // silu
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, long long ld, T* __restrict__ out, int I, long long n, int pairs, int act,
                                 float limit) {
    ti_pdl_trigger();
    ti_pdl_sync();
    gu = ti_dependent(gu);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
        const long long m = idx / I;
        const int i = (int)(idx - m * I);
        const T* row = gu + m * ld;
        const float g = to_f32(pairs ? row[2 * i] : row[i]);
        const float u = to_f32(pairs ? row[2 * i + 1] : row[I + i]);
        if (act == 2) {      // a clamped gate with a sharpened sigmoid, times the clamped up value plus one
            const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
            out[idx] = from_f32<T>(gc / (1.0f + expf(-1.702f * gc)) * (uc + 1.0f));
        } else {
            out[idx] = from_f32<T>(gate_act(g, act) * u);
        }
    }
}

}  // namespace

// gu: [M, 2 I] with row stride ld: gate in the first I columns and up in the rest, or with `pairs` gate_i and up_i side
// by side.  out: dense [M, I] = act(gate) * up, in 32-bit with one rounding.  act: 0 silu, 1 gelu (tanh form); 2:
// g' sigmoid(1.702 g') (u' + 1) with g' = min(gate, limit), u' = clamp(up, -limit, limit).
extern "C" int ti_gated_act(const void* gu, long long ld, void* out, int M, int I, int pairs, int act, float limit, int dtype,
                            cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && I > 0 && ld >= 2LL * I, "gated_act: bad sizes M=%d I=%d", M, I);
    TI_REQUIRE(act >= 0 && act <= 2, "gated_act: unknown activation %d", act);
    const long long n = (long long)M * I;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(gated_act_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (const T*)gu, ld, (T*)out, I, n, pairs, act, limit));
        TI_CHECK_LAUNCH("gated_act");
        return 0;
    });
}
