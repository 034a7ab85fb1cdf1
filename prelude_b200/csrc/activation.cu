// SiLU-gated product on a merged gate/up projection:
//   out[t, i] = silu(gu[t, i]) * gu[t, I + i],  silu(g) = g / (1 + exp(-g))
// computed in float32 (crates/prelude-cuda/src/kernels/kernels_src/elementwise/silu_mul.cu:27-32).
// The merged layout is the reference's gate_up projection, gate rows first
// (crates/prelude-core/src/models/qwen3.rs:411-447).
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n_tokens, int inter) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = n_tokens * inter;
    if (idx >= total) return;
    long long t = idx / inter;
    int i = (int)(idx % inter);
    float g = pb_ld(gu + t * 2 * inter + i);
    float u = pb_ld(gu + t * 2 * inter + inter + i);
    pb_st(out + idx, g / (1.0f + expf(-g)) * u);
}

// bfloat16, 8 elements per thread; inter % 8 == 0.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       long long n_tokens, int inter) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = inter / 8;
    if (idx >= n_tokens * per_row) return;
    long long t = idx / per_row;
    int c = (int)(idx % per_row) * 8;
    uint4 graw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c);
    uint4 uraw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 oraw;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = oraw;
}

PB_API int pb_silu_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && inter > 0, "silu_mul: bad sizes T=%d I=%d", n_tokens, inter);
    if (n_tokens == 0) return 0;
    const int threads = 256;
    if (dtype == PB_BF16 && inter % 8 == 0 && pb_aligned(gate_up, 16) && pb_aligned(out, 16)) {
        long long n = (long long)n_tokens * (inter / 8);
        pb_launch(silu_mul_bf16x8_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n_tokens, inter);
    } else {
        long long n = (long long)n_tokens * inter;
        PB_REQUIRE((n + threads - 1) / threads < (1ll << 31), "silu_mul: too many elements");
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(silu_mul_kernel<T>, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream, 
                (const T*)gate_up, (T*)out, n_tokens, inter)));
    }
    PB_CHECK_LAUNCH("silu_mul");
    return 0;
}

// Clamped gated unit on a merged gate/up projection:
//   a = min(gu[t, i], limit), b = clamp(gu[t, I + i], -limit, limit), out[t, i] = a * sigmoid(alpha * a) * (b + 1)
// in float32, rounded once.
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n_tokens, int inter,
                                   float limit, float alpha) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tokens * inter) return;
    long long t = idx / inter;
    int i = (int)(idx % inter);
    float a = fminf(pb_ld(gu + t * 2 * inter + i), limit);
    float b = fminf(fmaxf(pb_ld(gu + t * 2 * inter + inter + i), -limit), limit);
    pb_st(out + idx, a / (1.0f + expf(-alpha * a)) * (b + 1.0f));
}

PB_API int pb_clamped_glu(const void* gate_up, void* out, int dtype, int n_tokens, int inter, float limit, float alpha,
                          cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && inter > 0 && limit > 0.f, "clamped_glu: bad sizes T=%d I=%d limit=%g", n_tokens, inter, limit);
    if (n_tokens == 0) return 0;
    const int threads = 256;
    long long n = (long long)n_tokens * inter;
    PB_REQUIRE((n + threads - 1) / threads < (1ll << 31), "clamped_glu: too many elements");
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(clamped_glu_kernel<T>, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream,
            (const T*)gate_up, (T*)out, (long long)n_tokens, inter, limit, alpha)));
    PB_CHECK_LAUNCH("clamped_glu");
    return 0;
}


// tanh, element by element in float32 (the squashing between the two small products of a learned decay).
template <typename T>
__global__ void tanh_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pb_st(out + i, tanhf(pb_ld(x + i)));
}

PB_API int pb_tanh(const void* x, void* out, int dtype, long long n, cudaStream_t stream) {
    PB_REQUIRE(n >= 0 && x && out, "tanh: bad arguments");
    if (n == 0) return 0;
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(tanh_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const T*)x, (T*)out, n)));
    PB_CHECK_LAUNCH("tanh");
    return 0;
}


// GELU-gated product on a merged gate/up projection, the tanh form:
//   out[t, i] = gelu(gu[t, i]) * gu[t, I + i],  gelu(g) = 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))
// in float32, rounded once.
template <typename T>
__global__ void gelu_tanh_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n_tokens, int inter) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tokens * inter) return;
    long long t = idx / inter;
    int i = (int)(idx % inter);
    const float g = pb_ld(gu + t * 2 * inter + i);
    const float u = pb_ld(gu + t * 2 * inter + inter + i);
    pb_st(out + idx, pb_gelu_tanh(g) * u);
}

// bfloat16, 8 elements per thread; inter % 8 == 0.
__global__ void gelu_tanh_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                            long long n_tokens, int inter) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = inter / 8;
    if (idx >= n_tokens * per_row) return;
    long long t = idx / per_row;
    int c = (int)(idx % per_row) * 8;
    uint4 graw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c);
    uint4 uraw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 oraw;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        o2[k] = __floats2bfloat162_rn(pb_gelu_tanh(g.x) * u.x, pb_gelu_tanh(g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = oraw;
}

PB_API int pb_gelu_tanh_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && inter > 0, "gelu_tanh_mul: bad sizes T=%d I=%d", n_tokens, inter);
    if (n_tokens == 0) return 0;
    const int threads = 256;
    if (dtype == PB_BF16 && inter % 8 == 0 && pb_aligned(gate_up, 16) && pb_aligned(out, 16)) {
        long long n = (long long)n_tokens * (inter / 8);
        pb_launch(gelu_tanh_mul_bf16x8_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream,
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, (long long)n_tokens, inter);
    } else {
        long long n = (long long)n_tokens * inter;
        PB_REQUIRE((n + threads - 1) / threads < (1ll << 31), "gelu_tanh_mul: too many elements");
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(gelu_tanh_mul_kernel<T>, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream,
                (const T*)gate_up, (T*)out, (long long)n_tokens, inter)));
    }
    PB_CHECK_LAUNCH("gelu_tanh_mul");
    return 0;
}


// SiLU in place on the first `cols` columns of rows `ld` apart, float32 arithmetic, one rounding.
template <typename T>
__global__ void silu_cols_kernel(T* __restrict__ x, long long ld, long long n_tokens, int cols) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tokens * cols) return;
    T* p = x + (idx / cols) * ld + idx % cols;
    const float v = pb_ld(p);
    pb_st(p, v / (1.0f + expf(-v)));
}

// bfloat16, 8 elements per thread; cols % 8 == 0, ld % 8 == 0, x 16-byte aligned.
__global__ void silu_cols_bf16x8_kernel(__nv_bfloat16* __restrict__ x, long long ld, long long n_tokens, int cols) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = cols / 8;
    if (idx >= n_tokens * per_row) return;
    __nv_bfloat16* p = x + (idx / per_row) * ld + (idx % per_row) * 8;
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        h[k] = __floats2bfloat162_rn(f.x / (1.0f + expf(-f.x)), f.y / (1.0f + expf(-f.y)));
    }
    *reinterpret_cast<uint4*>(p) = raw;
}

PB_API int pb_silu_cols(void* x, long long ld, int dtype, int n_tokens, int cols, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && cols > 0 && ld >= cols && x, "silu_cols: bad arguments");
    if (n_tokens == 0) return 0;
    const int threads = 256;
    if (dtype == PB_BF16 && cols % 8 == 0 && ld % 8 == 0 && pb_aligned(x, 16)) {
        const long long n = (long long)n_tokens * (cols / 8);
        pb_launch(silu_cols_bf16x8_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream, (__nv_bfloat16*)x, ld,
                  (long long)n_tokens, cols);
    } else {
        const long long n = (long long)n_tokens * cols;
        PB_REQUIRE((n + threads - 1) / threads < (1ll << 31), "silu_cols: too many elements");
        PB_DISPATCH_DTYPE(dtype, T, (pb_launch(silu_cols_kernel<T>, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream,
                                               (T*)x, ld, (long long)n_tokens, cols)));
    }
    PB_CHECK_LAUNCH("silu_cols");
    return 0;
}
