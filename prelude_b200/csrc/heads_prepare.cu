// From a step's projections to queries ready for attention and keys and values in their pages, for mixers whose
// norm is per head with one scale shared by all heads, whose rotation (if any) is given by rates, whose keys and
// values may differ in size, and whose values may be blended with another layer's values of the same token.
//
// One block per token, one warp per head at a time.  In float32 throughout, one rounding at the store:
//   * optional RMS norm of every q head and every k head over its own elements, scale q_w / k_w [size of a head] or
//     none, before the rotation or after it (the two differ where the rotation's amplitude is not 1);
//   * rotation of the first `rot_dims` elements of every q and k head: angle = float(position) * rate[i]; `adjacent`
//     pairs element 2i with 2i + 1, otherwise i with i + rot_dims / 2; a pair (u, v) becomes
//     amplitude * (u cos - v sin, v cos + u sin);
//   * values: v <- (1 - mix) v + mix * v_other[t] where v_other is given ([T, Gv * vd] rows `ld_other` apart); the
//     unblended v is copied to v_copy where that is given (the layer whose values later layers blend with);
//   * queries to q_out [T, H, qd]; keys [G, kd] and values [Gv, vd] into the token's page (layout
//     [pages, heads, page_size, size]).
// A token whose row of the block table is negative is padding: nothing is read or written for it.
#include "common.cuh"

#include <math.h>

namespace {

// norm: 0 none; 1 before the rotation (what is rotated is x / rms(x) * w); 2 after it (rotated(x) / rms(rotated(x)) * w).
// A null w is a scale of ones.
template <typename T>
__device__ __forceinline__ void prepare_head(const T* __restrict__ in, T* __restrict__ out, int size, int norm, const float* __restrict__ w,
                                             float eps, const float* __restrict__ cs, int rot_dims, int adjacent, int lane) {
    float inv = 1.0f;
    if (norm == 1) {
        float ss = 0.f;
        for (int d = lane; d < size; d += 32) { const float v = pb_ld(in + d); ss += v * v; }
        inv = 1.0f / sqrtf(pb_warp_sum(ss) / (float)size + eps);
    }
    const bool scale_first = norm == 1 && w != nullptr;
    const int half = rot_dims >> 1;
    auto turned = [&](int d) {
        float own = pb_ld(in + d) * inv * (scale_first ? w[d] : 1.0f);
        if (d < rot_dims) {
            int i, partner;
            bool first;
            if (adjacent) { i = d >> 1; first = (d & 1) == 0; partner = first ? d + 1 : d - 1; }
            else { first = d < half; i = first ? d : d - half; partner = first ? d + half : d - half; }
            const float other = pb_ld(in + partner) * inv * (scale_first ? w[partner] : 1.0f);
            const float c = cs[2 * i], s = cs[2 * i + 1];
            own = first ? own * c - other * s : own * c + other * s;
        }
        return own;
    };
    if (norm == 2) {
        float ss = 0.f;
        for (int d = lane; d < size; d += 32) { const float v = turned(d); ss += v * v; }
        const float after = 1.0f / sqrtf(pb_warp_sum(ss) / (float)size + eps);
        for (int d = lane; d < size; d += 32) pb_st(out + d, turned(d) * after * (w ? w[d] : 1.0f));
        return;
    }
    for (int d = lane; d < size; d += 32) pb_st(out + d, turned(d));
}

template <typename T>
__global__ void heads_prepare_kernel(const T* __restrict__ q_in, long long ldq, const T* __restrict__ k_in, long long ldk,
                                     const T* __restrict__ v_in, long long ldv, const float* __restrict__ q_w,
                                     const float* __restrict__ k_w, int norm, float eps, const float* __restrict__ rates,
                                     float amplitude, int rot_dims, int adjacent, const T* __restrict__ v_other, T* __restrict__ v_copy,
                                     long long ld_other, float mix,
                                     const int32_t* __restrict__ positions, const int32_t* __restrict__ table_row,
                                     const int32_t* __restrict__ block_table, int table_stride, int page_size, int num_pages,
                                     T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int H, int qd, int G,
                                     int kd, int Gv, int vd, int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    extern __shared__ float cs[];                          // cosine and sine of the token's angles
    const int t = blockIdx.x;
    const int row = table_row[t];
    if (row < 0) return;
    const int p = positions[t];
    if (rates != nullptr) {
        for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
            float sn, c;
            sincosf((float)p * rates[i], &sn, &c);
            cs[2 * i] = c * amplitude;
            cs[2 * i + 1] = sn * amplitude;
        }
        __syncthreads();
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int rd = rates ? rot_dims : 0;
    for (int h = warp; h < H; h += nwarp)
        prepare_head(q_in + (size_t)t * ldq + (size_t)h * qd, q_out + ((size_t)t * H + h) * qd, qd, norm, q_w, eps, cs, rd, adjacent, lane);
    if (k_pages == nullptr) return;
    const int page = block_table[(size_t)row * table_stride + p / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
        return;
    }
    const int in_page = p % page_size;
    for (int g = warp; g < G; g += nwarp)
        prepare_head(k_in + (size_t)t * ldk + (size_t)g * kd, k_pages + (((size_t)page * G + g) * page_size + in_page) * kd, kd, norm, k_w, eps,
                     cs, rd, adjacent, lane);
    if (v_pages == nullptr || v_in == nullptr) return;
    const T* vv = v_in + (size_t)t * ldv;
    for (int i = threadIdx.x; i < Gv * vd; i += blockDim.x) {
        const int g = i / vd, d = i - g * vd;
        float v = pb_ld(vv + i);
        if (v_copy != nullptr) v_copy[(size_t)t * ld_other + i] = vv[i];
        if (v_other != nullptr) v = (1.0f - mix) * v + mix * pb_ld(v_other + (size_t)t * ld_other + i);
        pb_st(v_pages + (((size_t)page * Gv + g) * page_size + in_page) * vd + d, v);
    }
}

}  // namespace

// q_in [n_tokens, H * qd], k_in [n_tokens, G * kd], v_in [n_tokens, Gv * vd]: views with dense rows ldq, ldk, ldv apart;
// norm 0: none; 1: every q and k head brought to unit root mean square before the rotation; 2: after it; q_w [qd], k_w [kd]
// float32 scales of the norm, or null (ones); rates float32 [rot_dims / 2] or null (no rotation), cosine and sine
// both times `amplitude`; v_other, v_copy
// [n_tokens, Gv * vd] rows ld_other apart, or null; k_pages null: nothing is cached (then only the queries are made).
PB_API int pb_heads_prepare(const void* q_in, long long ldq, const void* k_in, long long ldk, const void* v_in, long long ldv, int dtype,
                            const float* q_w, const float* k_w, int norm, float eps, const float* rates, float amplitude, int rot_dims,
                            int adjacent,
                            const void* v_other, void* v_copy, long long ld_other, float mix, const int32_t* positions,
                            const int32_t* table_row, const int32_t* block_table, int table_stride, int page_size, int num_pages,
                            void* q_out, void* k_pages, void* v_pages, int n_tokens, int H, int qd, int G, int kd, int Gv, int vd,
                            int* status, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && H > 0 && qd > 0, "heads_prepare: bad sizes");
    PB_REQUIRE(q_in && q_out && positions && table_row, "heads_prepare: null pointer");
    PB_REQUIRE(norm >= 0 && norm <= 2 && (norm != 0 || (q_w == nullptr && k_w == nullptr)), "heads_prepare: norm %d", norm);
    PB_REQUIRE(rates == nullptr || (rot_dims > 0 && rot_dims % 2 == 0 && rot_dims <= qd && rot_dims <= 8192),
               "heads_prepare: a rotation of %d elements does not fit a head of %d", rot_dims, qd);
    if (k_pages != nullptr) {
        PB_REQUIRE(k_in && block_table && G > 0 && kd > 0 && page_size > 0 && num_pages > 0 && table_stride > 0,
                   "heads_prepare: keys need pages, tables and sizes");
        PB_REQUIRE(rates == nullptr || rot_dims <= kd, "heads_prepare: the rotation does not fit a key head");
        PB_REQUIRE(v_pages == nullptr || (v_in && Gv > 0 && vd > 0), "heads_prepare: values need sizes");
        PB_REQUIRE((v_other == nullptr && v_copy == nullptr) || (v_pages != nullptr && ld_other >= (long long)Gv * vd),
                   "heads_prepare: blended values need value pages and rows of %d", Gv * vd);
    }
    if (n_tokens == 0) return 0;
    // a warp per head at a time; a step of few tokens has few blocks, so each gets as many warps as the token has query
    // heads (they are the most), 4 to 16
    int threads = n_tokens < 128 ? 32 * H : 128;
    threads = threads < 128 ? 128 : (threads > 512 ? 512 : threads);
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(heads_prepare_kernel<T>, dim3(n_tokens), dim3(threads), rates ? (size_t)rot_dims * sizeof(float) : 0, stream, (const T*)q_in, ldq,
                   (const T*)k_in, ldk, (const T*)v_in, ldv, q_w, k_w, norm, eps, rates, amplitude, rot_dims, adjacent, (const T*)v_other, (T*)v_copy, ld_other, mix,
                   positions, table_row, block_table, table_stride, page_size, num_pages, (T*)q_out, (T*)k_pages, (T*)v_pages, H, qd, G, kd, Gv,
                   vd, status)));
    PB_CHECK_LAUNCH("heads_prepare");
    return 0;
}
