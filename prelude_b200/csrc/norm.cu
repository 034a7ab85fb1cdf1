// RMSNorm and fused residual-add + RMSNorm.
//
//   y = x / sqrt(mean(x^2) + eps) * w          (all arithmetic in float32)
//
// The residual stream `res` is float32 in every mode.  The fused form does
//   res += x ;  y = rmsnorm(res) * w
// in one pass over the row, which is the reference's add+norm protocol
// (crates/prelude-core/src/models/commons/linear.rs:471-488; kernels
// crates/prelude-cuda/src/kernels/kernels_src/normalization/rmsnorm.cu:33-51, 230-355)
// with the sum kept in 32-bit instead of being rounded to the model type.
//
// One block per row.  The block size depends on the row width only, so the
// order of the reduction, and with it every bit of the result, is the same
// whatever else is in the batch.
#include "common.cuh"


PB_TIMELINE_UNIT(norm)

__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = pb_warp_sum(v);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nwarp; ++i) total += smem[i];   // same order in every thread
    __syncthreads();
    return total;
}

template <typename TX, typename TY>
__global__ void add_rmsnorm_kernel(const TX* __restrict__ x, int n_parts, size_t part_stride, float* __restrict__ res,
                                   const float* __restrict__ w, TY* __restrict__ y, int width, float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    size_t row = blockIdx.x;
    float* r = res + row * width;
    TY* out = y + row * width;
    float ss = 0.f;
    if (x != nullptr) {
        const TX* xr = x + row * width;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = r[i];
            for (int s = 0; s < n_parts; ++s) v += pb_ld(xr + s * part_stride + i);     // the parts in ascending order
            r[i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = r[i];
            ss += v * v;
        }
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, r[i] * inv * w[i]);
}

// Four elements per thread and access, the row kept in registers between the
// two passes.  width % 4 == 0, width <= 4 * blockDim * ITERS.
// SCALED: what is added is xs times the parts' sum (taken on its own, in ascending order), as one fused multiply-add.
template <typename TX, typename TY, int ITERS, bool SCALED = false>
__global__ void add_rmsnorm_vec4_kernel(const TX* __restrict__ x, int n_parts, size_t part_stride, float* __restrict__ res,
                                        const float* __restrict__ w, TY* __restrict__ y, int width, float eps, float xs) {
    pb_grid_dep_launch();
    PB_TL(PB_TL_NORM, PB_TL_ENTRY);
    __shared__ float red[32];
    size_t row = blockIdx.x;
    float4* r4 = reinterpret_cast<float4*>(res + row * width);
    const int n4 = width >> 2;
    // the scale is written by no kernel: it is fetched while the kernel before this one is still running
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4 scale[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) scale[it] = w4[i];
    }
    pb_grid_dep_wait();
    PB_TL(PB_TL_NORM, PB_TL_AFTER_WAIT);
    float4 keep[ITERS];
    float ss = 0.f;
    // Every load of the row is issued before the first sum (up to four parts): the kernel is one round trip to
    // the L2 cache, a reduction and a store, and with the loads of one iteration behind the store of the one
    // before it was three round trips (4.1 us for 8 rows of 2,560 in a decode step).
    float4 part[ITERS][4];
    uint2 raw[ITERS];
    const bool ahead = x != nullptr && (sizeof(TX) == 2 || n_parts <= 4);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            keep[it] = r4[i];
            if (ahead) {
                const TX* xr = x + row * width + 4 * (size_t)i;
                if constexpr (sizeof(TX) == 2) {
                    raw[it] = *reinterpret_cast<const uint2*>(xr);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        part[it][u] = (u < n_parts) ? *reinterpret_cast<const float4*>(xr + (size_t)u * part_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            float4 v = keep[it];
            if (x != nullptr) {
                float4 acc = SCALED ? make_float4(0.f, 0.f, 0.f, 0.f) : v;
                const TX* xr = x + row * width + 4 * (size_t)i;
                if constexpr (sizeof(TX) == 2) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[it]);
                    float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
                    acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
                } else if (ahead) {
                    // the parts in ascending order
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (u < n_parts) { acc.x += part[it][u].x; acc.y += part[it][u].y; acc.z += part[it][u].z; acc.w += part[it][u].w; }
                } else {
                    // the parts in ascending order, four loads in flight at a time
                    for (int s0 = 0; s0 < n_parts; s0 += 4) {
                        float4 a[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            a[u] = (s0 + u < n_parts) ? *reinterpret_cast<const float4*>(xr + (size_t)(s0 + u) * part_stride)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (s0 + u < n_parts) { acc.x += a[u].x; acc.y += a[u].y; acc.z += a[u].z; acc.w += a[u].w; }
                    }
                }
                if constexpr (SCALED) v = make_float4(fmaf(xs, acc.x, v.x), fmaf(xs, acc.y, v.y), fmaf(xs, acc.z, v.z), fmaf(xs, acc.w, v.w));
                else v = acc;
                r4[i] = v;
            }
            keep[it] = v;
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            float4 v = keep[it], g = scale[it];
            float o0 = v.x * inv * g.x, o1 = v.y * inv * g.y, o2 = v.z * inv * g.z, o3 = v.w * inv * g.w;
            TY* out = y + row * width + 4 * (size_t)i;
            if constexpr (sizeof(TY) == 2) {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
                uint2 raw;
                raw.x = *reinterpret_cast<uint32_t*>(&p0);
                raw.y = *reinterpret_cast<uint32_t*>(&p1);
                *reinterpret_cast<uint2*>(out) = raw;
            } else {
                *reinterpret_cast<float4*>(out) = make_float4(o0, o1, o2, o3);
            }
        }
    }
    PB_TL(PB_TL_NORM, PB_TL_DONE);
}

static int norm_threads(int width) {
    if (width <= 64) return 32;
    if (width <= 512) return 64;
    if (width <= 2048) return 128;
    return 256;
}

template <typename TX, typename TY>
static int launch_add_rmsnorm(const void* x, int n_parts, size_t part_stride, float* res, const float* w, void* y, int rows,
                              int width, float eps, cudaStream_t stream) {
    int threads = norm_threads(width);
    bool vec = width % 4 == 0 && pb_aligned(res, 16) && pb_aligned(w, 16) && pb_aligned(y, 8 * sizeof(TY) / 2) &&
               (x == nullptr || (pb_aligned(x, 8 * sizeof(TX) / 2) && part_stride % 4 == 0)) && width <= 4 * threads * 8;
    if (vec) {
        int iters = (width / 4 + threads - 1) / threads;
        if (iters <= 2)
            pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 2>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps, 1.0f);
        else if (iters <= 4)
            pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 4>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps, 1.0f);
        else
            pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 8>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps, 1.0f);
    } else {
        pb_launch(add_rmsnorm_kernel<TX, TY>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps);
    }
    return 0;
}

// res[rows, width] float32 (updated in place when x is given); x may be null
// (no add); w float32 [width]; y [rows, width] of type dtype.  x has type dtype,
// or, with x_parts > 0, it is x_parts float32 arrays [rows, width], part_stride
// elements apart, whose sum is what is added (the partial sums of a product
// whose K was cut into parts).
PB_API int pb_add_rmsnorm(const void* x, int x_parts, long long part_stride, float* res, const float* w, void* y, int dtype,
                          int rows, int width, float eps, cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && width > 0, "add_rmsnorm: bad sizes rows=%d width=%d", rows, width);
    PB_REQUIRE(res && w && y, "add_rmsnorm: null pointer");
    PB_REQUIRE(x_parts >= 0 && x_parts <= 64 && (x_parts == 0 || (x && part_stride >= (long long)rows * width)),
               "add_rmsnorm: %d parts %lld apart", x_parts, part_stride);
    if (rows == 0) return 0;
    if (x_parts > 0) {
        PB_DISPATCH_DTYPE(dtype, T, (launch_add_rmsnorm<float, T>(x, x_parts, (size_t)part_stride, res, w, y, rows, width, eps, stream)));
    } else {
        PB_DISPATCH_DTYPE(dtype, T, (launch_add_rmsnorm<T, T>(x, 1, 0, res, w, y, rows, width, eps, stream)));
    }
    PB_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// Final norm on chosen rows only: y[i] = rmsnorm(res[rows[i]] + x[rows[i]]) * w.
// The residual stream is left as it is; only the rows whose logits are wanted
// are normalised (the reference selects the last row of each request after the
// final norm, crates/prelude-core/src/models/commons/mod.rs:227-243; the order
// does not change the values).
template <typename TX, typename TY>
__global__ void gather_add_rmsnorm_kernel(const TX* __restrict__ x, int n_parts, size_t part_stride,
                                          const float* __restrict__ res, const int32_t* __restrict__ rows,
                                          const float* __restrict__ w, TY* __restrict__ y, int width, int n_rows_total,
                                          float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    const int src = rows[blockIdx.x];
    TY* out = y + (size_t)blockIdx.x * width;
    if (src < 0 || src >= n_rows_total) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, 0.f);
        return;
    }
    const float* r = res + (size_t)src * width;
    const TX* xr = x ? x + (size_t)src * width : nullptr;
    auto value = [&](int i) {
        float v = r[i];
        if (xr) for (int s = 0; s < n_parts; ++s) v += pb_ld(xr + s * part_stride + i);   // the parts in ascending order
        return v;
    };
    // a thread's elements stay in registers between the two passes where the row is short enough (16 per thread:
    // rows of up to 4,096 at 256 threads); the loads of the first pass are independent of one another
    constexpr int KEEP = 16;
    float kept[KEEP];
    const bool fits = width <= KEEP * (int)blockDim.x;
    float ss = 0.f;
    if (fits) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            kept[k] = i < width ? value(i) : 0.f;
            ss += kept[k] * kept[k];
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = value(i);
            ss += v * v;
        }
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
    if (fits) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < width) pb_st(out + i, kept[k] * inv * w[i]);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, value(i) * inv * w[i]);
    }
}

// x as for pb_add_rmsnorm: of type dtype, or x_parts float32 arrays to be added up.
PB_API int pb_gather_add_rmsnorm(const void* x, int x_parts, long long part_stride, const float* res, const int32_t* rows,
                                 const float* w, void* y, int dtype, int n_out, int n_rows_total, int width, float eps,
                                 cudaStream_t stream) {
    PB_REQUIRE(n_out >= 0 && width > 0 && n_rows_total >= 0, "gather_add_rmsnorm: bad sizes");
    PB_REQUIRE(res && rows && w && y, "gather_add_rmsnorm: null pointer");
    PB_REQUIRE(x_parts >= 0 && x_parts <= 64 && (x_parts == 0 || (x && part_stride >= (long long)n_rows_total * width)),
               "gather_add_rmsnorm: %d parts %lld apart", x_parts, part_stride);
    if (n_out == 0) return 0;
    if (x_parts > 0) {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(gather_add_rmsnorm_kernel<float, T>, dim3(n_out), dim3(norm_threads(width)), 0, stream,
                (const float*)x, x_parts, (size_t)part_stride, res, rows, w, (T*)y, width, n_rows_total, eps)));
    } else {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(gather_add_rmsnorm_kernel<T, T>, dim3(n_out), dim3(norm_threads(width)), 0, stream,
                (const T*)x, 1, (size_t)0, res, rows, w, (T*)y, width, n_rows_total, eps)));
    }
    PB_CHECK_LAUNCH("gather_add_rmsnorm");
    return 0;
}

// Plain norm of a tensor of the model's own type (used by parts that are not
// on the residual stream, and by the per-kernel tests).
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ y, int width,
                               float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    size_t row = blockIdx.x;
    const T* xr = x + row * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = pb_ld(xr + i);
        ss += v * v;
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(y + row * width + i, pb_ld(xr + i) * inv * w[i]);
}

PB_API int pb_rmsnorm(const void* x, const float* w, void* y, int dtype, int rows, int width, float eps,
                      cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
    PB_REQUIRE(x && w && y, "rmsnorm: null pointer");
    if (rows == 0) return 0;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(rmsnorm_kernel<T>, dim3(rows), dim3(norm_threads(width)), 0, stream, (const T*)x, w, (T*)y, width, eps)));
    PB_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// A sublayer's output that is normed before it joins the residual stream, fused with the norm that follows:
//   res += x / sqrt(mean(x^2) + eps_x) * wx ;  y = res / sqrt(mean(res^2) + eps) * w
// one block per row, all in float32; x is rounded nowhere between its norm and the sum.  Without w and y only the
// sum is made.  With `rows` (the gather form) row i of y is made from row rows[i] of x and res, and res is left alone.
// The row is kept in shared memory between the passes where it fits, else it is read again.
template <typename TX, typename TY>
__global__ void normed_add_rmsnorm_kernel(const TX* __restrict__ x, const float* __restrict__ wx, float eps_x,
                                          float* __restrict__ res, const int32_t* __restrict__ rows, int n_rows_total,
                                          const float* __restrict__ w, TY* __restrict__ y, int width, float eps, int keep) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    extern __shared__ float row_s[];
    __shared__ float red[32];
    const long long src = rows ? (long long)rows[blockIdx.x] : (long long)blockIdx.x;
    TY* out = y ? y + (size_t)blockIdx.x * width : nullptr;
    if (src < 0 || src >= n_rows_total) {
        if (out) for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, 0.f);
        return;
    }
    const TX* xr = x + (size_t)src * width;
    float* r = res + (size_t)src * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = pb_ld(xr + i);
        if (keep) row_s[i] = v;
        ss += v * v;
    }
    const float inv_x = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps_x);
    ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = r[i] + (keep ? row_s[i] : pb_ld(xr + i)) * inv_x * wx[i];
        if (rows == nullptr) r[i] = v;
        if (keep) row_s[i] = v;
        ss += v * v;
    }
    if (out == nullptr) return;
    // without a scale for the second norm there is none: the sum itself goes out, in the output's type
    const float inv = w ? 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps) : 1.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = keep ? row_s[i] : (rows == nullptr ? r[i] : r[i] + pb_ld(xr + i) * inv_x * wx[i]);
        pb_st(out + i, w ? v * inv * w[i] : v);
    }
}

// The same, four elements per thread and access, all loads of the row issued before the first sum and the row kept in
// registers between the passes; for every row of the stream, or (with `rows`) for the chosen rows, whose sum is not
// stored.  width % 4 == 0, width <= 4 * blockDim * ITERS.
template <typename TX, typename TY, int ITERS>
__global__ void normed_add_rmsnorm_vec4_kernel(const TX* __restrict__ x, const float* __restrict__ wx, float eps_x,
                                               float* __restrict__ res, const int32_t* __restrict__ rows, int n_rows_total,
                                               const float* __restrict__ w, TY* __restrict__ y, int width, float eps) {
    pb_grid_dep_launch();
    __shared__ float red[32];
    const int n4 = width >> 2;
    float4 gx[ITERS], gw[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {                     // the scales are written by no kernel: fetched before the wait
        const int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            gx[it] = reinterpret_cast<const float4*>(wx)[i];
            if (w) gw[it] = reinterpret_cast<const float4*>(w)[i];
        }
    }
    pb_grid_dep_wait();
    size_t row = blockIdx.x;
    if (rows != nullptr) {
        const int r = rows[blockIdx.x];
        if (r < 0 || r >= n_rows_total) return;
        row = (size_t)r;
    }
    float4 xv[ITERS], rv[ITERS];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            rv[it] = reinterpret_cast<const float4*>(res + row * width)[i];
            const TX* xr = x + row * width + 4 * (size_t)i;
            if constexpr (sizeof(TX) == 2) {
                const uint2 raw = *reinterpret_cast<const uint2*>(xr);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
                xv[it] = make_float4(a.x, a.y, b.x, b.y);
            } else {
                xv[it] = *reinterpret_cast<const float4*>(xr);
            }
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i < n4) { ss += xv[it].x * xv[it].x; ss += xv[it].y * xv[it].y; ss += xv[it].z * xv[it].z; ss += xv[it].w * xv[it].w; }
    }
    const float inv_x = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps_x);
    ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            float4 v = rv[it];
            v.x += xv[it].x * inv_x * gx[it].x; v.y += xv[it].y * inv_x * gx[it].y;
            v.z += xv[it].z * inv_x * gx[it].z; v.w += xv[it].w * inv_x * gx[it].w;
            if (rows == nullptr) reinterpret_cast<float4*>(res + row * width)[i] = v;
            rv[it] = v;
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
    }
    if (y == nullptr) return;
    const float inv = w ? 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps) : 1.0f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            const float4 v = rv[it], g = w ? gw[it] : make_float4(1.f, 1.f, 1.f, 1.f);
            const float o0 = w ? v.x * inv * g.x : v.x, o1 = w ? v.y * inv * g.y : v.y, o2 = w ? v.z * inv * g.z : v.z,
                        o3 = w ? v.w * inv * g.w : v.w;
            TY* out = y + (size_t)blockIdx.x * width + 4 * (size_t)i;       // chosen rows are stored one below the other
            if constexpr (sizeof(TY) == 2) {
                const __nv_bfloat162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
                uint2 raw;
                raw.x = *reinterpret_cast<const uint32_t*>(&p0);
                raw.y = *reinterpret_cast<const uint32_t*>(&p1);
                *reinterpret_cast<uint2*>(out) = raw;
            } else {
                *reinterpret_cast<float4*>(out) = make_float4(o0, o1, o2, o3);
            }
        }
    }
}

// x [n_rows_total, width] of type dtype; wx, w float32 [width]; res float32 [n_rows_total, width]; rows null (every
// row, res updated) or int32 [n_out] (those rows, res untouched); y [n_out, width] of type dtype, or null with w.
PB_API int pb_normed_add_rmsnorm(const void* x, const float* wx, float eps_x, float* res, const int32_t* rows, int n_out,
                                 int n_rows_total, const float* w, void* y, int dtype, int width, float eps,
                                 cudaStream_t stream) {
    PB_REQUIRE(n_out >= 0 && n_rows_total >= 0 && width > 0, "normed_add_rmsnorm: bad sizes");
    PB_REQUIRE(x && wx && res && (w == nullptr || y != nullptr), "normed_add_rmsnorm: null pointer");
    PB_REQUIRE(rows == nullptr ? n_out == n_rows_total : y != nullptr, "normed_add_rmsnorm: rows and outputs do not fit");
    if (n_out == 0) return 0;
    const int threads = norm_threads(width);
    const size_t esz = dtype == PB_BF16 ? 2 : 4;
    if (width % 4 == 0 && width <= 4 * threads * 8 && pb_aligned(x, 4 * esz) && pb_aligned(wx, 16) && pb_aligned(res, 16) &&
        (w == nullptr || pb_aligned(w, 16)) && (y == nullptr || pb_aligned(y, 4 * esz))) {
        const int iters = (width / 4 + threads - 1) / threads;
#define NA_VEC(IT)                                                                                                              \
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(normed_add_rmsnorm_vec4_kernel<T, T, IT>, dim3(n_out), dim3(threads), 0, stream, (const T*)x, wx, \
                                           eps_x, res, rows, n_rows_total, w, (T*)y, width, eps)))
        if (iters <= 2) NA_VEC(2);
        else if (iters <= 4) NA_VEC(4);
        else NA_VEC(8);
#undef NA_VEC
        PB_CHECK_LAUNCH("normed_add_rmsnorm");
        return 0;
    }
    const int keep = (size_t)width * sizeof(float) <= 40 * 1024 ? 1 : 0;
    const size_t smem = keep ? (size_t)width * sizeof(float) : 0;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(normed_add_rmsnorm_kernel<T, T>, dim3(n_out), dim3(norm_threads(width)), smem, stream, (const T*)x, wx, eps_x,
                   res, rows, n_rows_total, w, (T*)y, width, eps, keep)));
    PB_CHECK_LAUNCH("normed_add_rmsnorm");
    return 0;
}


// A sublayer's output that joins the residual stream times a constant: res += scale * x ; y = rmsnorm(res) * w, one
// block per row, float32.  With `rows` only the chosen rows are made and res is left alone (the final norm at the
// places whose logits are wanted).  x as for pb_add_rmsnorm: of type dtype, or x_parts float32 arrays whose sum,
// taken in ascending order, is what is scaled and added.
template <typename TX, typename TY>
__global__ void scaled_add_rmsnorm_kernel(const TX* __restrict__ x, int n_parts, size_t part_stride, float scale, float* __restrict__ res,
                                          const int32_t* __restrict__ rows, int n_rows_total, const float* __restrict__ w,
                                          TY* __restrict__ y, int width, float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    const int src = rows ? rows[blockIdx.x] : (int)blockIdx.x;
    TY* out = y + (size_t)blockIdx.x * width;
    if (src < 0 || src >= n_rows_total) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, 0.f);
        return;
    }
    float* r = res + (size_t)src * width;
    const TX* xr = x + (size_t)src * width;
    auto value = [&](int i) {
        float a = pb_ld(xr + i);
        for (int s = 1; s < n_parts; ++s) a += pb_ld(xr + s * part_stride + i);
        return fmaf(scale, a, r[i]);
    };
    constexpr int KEEP = 16;
    float kept[KEEP];
    const bool fits = width <= KEEP * (int)blockDim.x;
    float ss = 0.f;
    if (fits) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            kept[k] = i < width ? value(i) : 0.f;
            ss += kept[k] * kept[k];
        }
        if (rows == nullptr) {
#pragma unroll
            for (int k = 0; k < KEEP; ++k) {
                const int i = threadIdx.x + k * blockDim.x;
                if (i < width) r[i] = kept[k];
            }
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = value(i);
            if (rows == nullptr) r[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    if (fits) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < width) pb_st(out + i, kept[k] * inv * w[i]);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, (rows ? value(i) : r[i]) * inv * w[i]);
    }
}

// The whole-step form on the vectorised kernel; false: the shape or the alignment is not taken.
template <typename TX, typename TY>
static bool launch_scaled_add_rmsnorm_vec4(const void* x, int n_parts, size_t part_stride, float xs, float* res, const float* w, void* y,
                                           int rows, int width, float eps, cudaStream_t stream) {
    const int threads = norm_threads(width);
    const bool vec = width % 4 == 0 && pb_aligned(res, 16) && pb_aligned(w, 16) && pb_aligned(y, 8 * sizeof(TY) / 2) &&
                     pb_aligned(x, 8 * sizeof(TX) / 2) && part_stride % 4 == 0 && width <= 4 * threads * 8;
    if (!vec) return false;
    const int iters = (width / 4 + threads - 1) / threads;
    if (iters <= 2)
        pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 2, true>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps, xs);
    else if (iters <= 4)
        pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 4, true>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps, xs);
    else
        pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 8, true>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps, xs);
    return true;
}

PB_API int pb_scaled_add_rmsnorm(const void* x, int x_parts, long long part_stride, float scale, float* res, const int32_t* rows,
                                 int n_out, int n_rows_total, const float* w, void* y, int dtype, int width, float eps,
                                 cudaStream_t stream) {
    PB_REQUIRE(n_out >= 0 && width > 0 && n_rows_total >= 0, "scaled_add_rmsnorm: bad sizes");
    PB_REQUIRE(x && res && w && y, "scaled_add_rmsnorm: null pointer");
    PB_REQUIRE(x_parts >= 0 && x_parts <= 64 && (x_parts == 0 || part_stride >= (long long)n_rows_total * width),
               "scaled_add_rmsnorm: %d parts %lld apart", x_parts, part_stride);
    PB_REQUIRE(rows != nullptr || n_out == n_rows_total, "scaled_add_rmsnorm: without chosen rows every row is made");
    if (n_out == 0) return 0;
    if (rows == nullptr) {
        bool done = false;
        if (x_parts > 0) {
            PB_DISPATCH_DTYPE(dtype, T, (done = launch_scaled_add_rmsnorm_vec4<float, T>(x, x_parts, (size_t)part_stride, scale, res, w, y, n_out, width, eps, stream)));
        } else {
            PB_DISPATCH_DTYPE(dtype, T, (done = launch_scaled_add_rmsnorm_vec4<T, T>(x, 1, (size_t)0, scale, res, w, y, n_out, width, eps, stream)));
        }
        if (done) {
            PB_CHECK_LAUNCH("scaled_add_rmsnorm");
            return 0;
        }
    }
    if (x_parts > 0) {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(scaled_add_rmsnorm_kernel<float, T>, dim3(n_out), dim3(norm_threads(width)), 0, stream, (const float*)x, x_parts,
                       (size_t)part_stride, scale, res, rows, n_rows_total, w, (T*)y, width, eps)));
    } else {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(scaled_add_rmsnorm_kernel<T, T>, dim3(n_out), dim3(norm_threads(width)), 0, stream, (const T*)x, 1, (size_t)0, scale,
                       res, rows, n_rows_total, w, (T*)y, width, eps)));
    }
    PB_CHECK_LAUNCH("scaled_add_rmsnorm");
    return 0;
}

// Two outputs side by side, each brought to unit root mean square over the row and scaled, then added:
// out = sa * a / rms(a) * wa + sb * b / rms(b) * wb, computed and handed out in float32 (what the residual add takes as
// a sum of one part).  One block per row.
template <typename T>
__global__ void normed_pair_sum_kernel(const T* __restrict__ a, const float* __restrict__ wa, float sa, const T* __restrict__ b,
                                       const float* __restrict__ wb, float sb, float eps, float* __restrict__ out, int width) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const T* ar = a + row * width;
    const T* br = b + row * width;
    float ssa = 0.f, ssb = 0.f;
#pragma unroll 8
    for (int i = threadIdx.x; i < width; i += blockDim.x) {          // several rounds' loads in flight together
        const float va = pb_ld(ar + i), vb = pb_ld(br + i);
        ssa += va * va;
        ssb += vb * vb;
    }
    const float ta = block_sum(ssa, red), tb = block_sum(ssb, red);
    const float ia = sa / sqrtf(ta / (float)width + eps), ib = sb / sqrtf(tb / (float)width + eps);
#pragma unroll 8
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        out[row * width + i] = pb_ld(ar + i) * ia * wa[i] + pb_ld(br + i) * ib * wb[i];
}

PB_API int pb_normed_pair_sum(const void* a, const float* wa, float sa, const void* b, const float* wb, float sb, float eps, float* out,
                              int dtype, int rows, int width, cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && width > 0, "normed_pair_sum: bad sizes");
    PB_REQUIRE(a && wa && b && wb && out, "normed_pair_sum: null pointer");
    if (rows == 0) return 0;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(normed_pair_sum_kernel<T>, dim3(rows), dim3(norm_threads(width)), 0, stream, (const T*)a, wa, sa, (const T*)b, wb, sb, eps,
                   out, width)));
    PB_CHECK_LAUNCH("normed_pair_sum");
    return 0;
}
