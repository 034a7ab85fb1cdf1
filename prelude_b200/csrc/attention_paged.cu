// Paged softmax attention with the options that designs combine, float32 arithmetic throughout: keys and
// values of different sizes, values that are the first `vd` elements of the cached key rows (a latent that is
// key and value at once), a window, first tokens that stay visible behind the window, chunks (a query sees only the
// keys of its own run of `chunk` positions), capped scores (cap * tanh(score / cap)), a learned sink per head whose
// exponential joins the denominator, and a gate per (token, head) whose sigmoid multiplies the head's output.
//
// One warp per (query token, query head).  A query at absolute position p of its request sees the keys at
// lo .. p with lo = max(0, p - window + 1) under a window, lo = p - p % chunk under chunks, else 0, and under a window
// also the keys at 0 .. keep_first - 1; all of them are in the cache because a step writes its keys before it attends.
// Keys are visited in blocks of 32 aligned to absolute positions, in ascending order, with a running maximum and
// sum; every lane scores one key (16-byte loads of its row), then all lanes add up the block's value rows.  The
// blocks, and so the order of every floating-point operation, depend on the query's position and the window only:
// not on how the tokens were cut into steps, not on the batch, not on the pages.
//
// It is the attention of the 32-bit path for these options and, in bfloat16, of the shapes the tensor-core kernel
// (attention_paged_tc.cu) does not take.
#include "common.cuh"

#include <math.h>

#define AP_WARPS 4
#define AP_MAX_VD 1024

namespace {

template <typename T> struct Chunk;
template <> struct Chunk<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
    }
};

template <typename T, int VPL>
__global__ void attention_paged_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                       T* __restrict__ out, const float* __restrict__ sink, const int32_t* __restrict__ positions,
                                       const int32_t* __restrict__ table_row, const int32_t* __restrict__ block_table,
                                       int table_stride, int page_size, int num_pages, int n_tokens, int H, int G, int kd, int vd,
                                       int v_row, int Gv, float scale, int window, int keep_first, int chunk, float softcap,
                                       const T* __restrict__ gate, long long ld_gate, int swizzle_k, int swizzle_v, int vec,
                                       int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    extern __shared__ float q_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* q_s = q_all + (size_t)warp * kd;
    const long long item = (long long)blockIdx.x * AP_WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int row = table_row[t];
    if (row < 0) return;
    const int kvh = h / (H / G), vh = Gv == G ? kvh : h / (H / Gv);
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : (chunk > 0 ? pos - pos % chunk : 0);
    const int kept = window > 0 ? min(keep_first, lo) : 0;          // first tokens the window has passed and that stay visible
    const int32_t* table = block_table + (size_t)row * table_stride;

    const T* qrow = q + ((size_t)t * H + h) * kd;
    for (int i = lane; i < kd; i += 32) q_s[i] = pb_ld(qrow + i);
    __syncwarp();

    float o[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool bad = false;
    constexpr int CN = Chunk<T>::N;

    // two runs of keys in ascending order: the kept first tokens (positions 0 .. kept - 1), then lo .. pos
    for (int run = kept > 0 ? 0 : 1; run < 2; ++run) {
    const int r_lo = run == 0 ? 0 : lo, r_hi = run == 0 ? kept - 1 : pos;
    for (int base = (r_lo / 32) * 32; base <= r_hi; base += 32) {
        const int j = base + lane;
        const bool valid = j >= r_lo && j <= r_hi;
        float s = -INFINITY;
        int page = -1;
        if (valid) {
            page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                bad = true;
                page = -1;
            } else {
                const int in_page = j % page_size;
                const T* kr = k_pages + (((size_t)page * G + kvh) * page_size + in_page) * kd;
                float acc = 0.f;
                if (vec) {
                    for (int c = 0; c < kd / CN; ++c) {
                        float e[CN];
                        Chunk<T>::load(kr + (swizzle_k ? ((c ^ (in_page & 7)) * CN) : c * CN), e);
#pragma unroll
                        for (int u = 0; u < CN; ++u) acc = fmaf(q_s[c * CN + u], e[u], acc);
                    }
                } else {
                    for (int d = 0; d < kd; ++d) acc = fmaf(q_s[d], pb_ld(kr + pb_kv_elem_offset(d, in_page, swizzle_k)), acc);
                }
                s = acc * scale;
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            }
        }
        const float bm = pb_warp_max(s);
        const float m_new = fmaxf(m, bm);
        if (m_new == -INFINITY) continue;   // only when every page id of the block was bad
        const float p = (page >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + pb_warp_sum(p);
#pragma unroll
        for (int i = 0; i < VPL; ++i) o[i] *= corr;
        const int n_in_block = min(32, r_hi - base + 1);
        for (int jj = 0; jj < n_in_block; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int pg = __shfl_sync(0xffffffffu, page, jj);
            if (pg < 0) continue;
            const int vin = (base + jj) % page_size;
            const T* vr = v_pages + (((size_t)pg * Gv + vh) * page_size + vin) * v_row;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) o[i] = fmaf(pj, pb_ld(vr + pb_kv_elem_offset(d, vin, swizzle_v)), o[i]);
            }
        }
        m = m_new;
    }
    }
    if (sink != nullptr) {                  // the sink: one more term of the denominator, no key, no value
        const float sk = sink[h];
        const float m_new = fmaxf(m, sk);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < VPL; ++i) o[i] *= corr;
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0 && status) atomicExch(status, 4);
    T* orow = out + ((size_t)t * H + h) * vd;
    float inv = l > 0.f ? 1.0f / l : 0.f;
    if (gate != nullptr) inv *= 1.0f / (1.0f + expf(-pb_ld(gate + (size_t)t * ld_gate + h)));
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) pb_st(orow + d, o[i] * inv);
    }
}

}  // namespace

// q [n_tokens, H, kd]; out [n_tokens, H, vd]; k_pages [num_pages, G, page_size, kd]; v_pages [num_pages, Gv, page_size,
// v_row] of which the first vd elements of a row are the value (v_pages == k_pages, v_row == kd, Gv == G: the values
// are the keys' first vd elements); sink float32 [H] or null; positions, table_row [n_tokens] (a negative row: padding);
// block_table [rows, table_stride]; window <= 0: no window; keep_first: positions below it stay visible behind the window;
// chunk > 0 (without a window): only keys of the query's own run of `chunk` positions; softcap > 0: scores capped;
// gate [n_tokens, H] with row stride ld_gate (columns of a projection) or null.
PB_API int pb_attention_paged(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype, const float* sink,
                              const int32_t* positions, const int32_t* table_row, const int32_t* block_table, int table_stride,
                              int page_size, int num_pages, int n_tokens, int H, int G, int kd, int vd, int v_row, int Gv,
                              float scale, int window, int keep_first, int chunk, float softcap, const void* gate, long long ld_gate,
                              int swizzle_k, int swizzle_v, int* status, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && Gv > 0 && H % G == 0 && H % Gv == 0,
               "attention_paged: %d query heads over %d key and %d value heads", H, G, Gv);
    PB_REQUIRE(kd > 0 && vd > 0 && vd <= AP_MAX_VD && v_row >= vd, "attention_paged: sizes kd=%d vd=%d (at most %d) row=%d", kd, vd,
               AP_MAX_VD, v_row);
    PB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "attention_paged: bad cache geometry");
    PB_REQUIRE(keep_first >= 0 && chunk >= 0 && !(window > 0 && chunk > 0) && (gate == nullptr || ld_gate >= H),
               "attention_paged: window %d, kept %d, chunk %d", window, keep_first, chunk);
    PB_REQUIRE((!swizzle_k || kd % 8 == 0) && (!swizzle_v || v_row % 8 == 0), "attention_paged: permuted rows need sizes in multiples of 8");
    const size_t smem = (size_t)AP_WARPS * kd * sizeof(float);
    PB_REQUIRE(smem <= 48 * 1024, "attention_paged: keys of %d elements do not fit", kd);
    if (n_tokens == 0) return 0;
    const long long items = (long long)n_tokens * H;
    const long long blocks = (items + AP_WARPS - 1) / AP_WARPS;
    PB_REQUIRE(blocks < (1ll << 31), "attention_paged: too many rows");
    const int piece = dtype == PB_BF16 ? 8 : 4;
    const int vec = (kd % piece == 0 && pb_aligned(k_pages, 16)) ? 1 : 0;
#define AP_LAUNCH(VPL)                                                                                                        \
    PB_DISPATCH_DTYPE(dtype, T,                                                                                               \
        (pb_launch(attention_paged_kernel<T, VPL>, dim3((unsigned)blocks), dim3(AP_WARPS * 32), smem, stream, (const T*)q,     \
                   (const T*)k_pages, (const T*)v_pages, (T*)out, sink, positions, table_row, block_table, table_stride,       \
                   page_size, num_pages, n_tokens, H, G, kd, vd, v_row, Gv, scale, window, keep_first, chunk, softcap, (const T*)gate, ld_gate,  \
                   swizzle_k, swizzle_v, vec, status)))
    if (vd <= 64) AP_LAUNCH(2);
    else if (vd <= 128) AP_LAUNCH(4);
    else if (vd <= 256) AP_LAUNCH(8);
    else if (vd <= 512) AP_LAUNCH(16);
    else AP_LAUNCH(32);
#undef AP_LAUNCH
    PB_CHECK_LAUNCH("attention_paged");
    return 0;
}
