// Time mixing with a decaying matrix state per head and a bonus for the current token:
//
//   pb_token_shift_mix   out[s][t] = x_t + (x_(t-1) - x_t) * mu[s] for each of `n_mix` learned blends mu; x_(t-1) is the
//                        previous token of the same sequence: the row above inside a step, the sequence's carried row
//                        for the first token of a step, zeros at position 0
//   pb_wkv_scan          per head, token by token, with the state S [dim (key channel), dim (value)] in float32:
//                            w = exp(-exp(w_raw + w0))                       (per key channel)
//                            o = (S + diag(u) k v^T)^T r  =  S^T r + (sum_n r_n u_n k_n) v
//                            S <- diag(w) S + k v^T
//
// Decay and its exponentials, the state and every sum over it are float32 whatever the run's type; r, k, v and w_raw
// (projections) are of the run's type.  A sequence's tokens are visited in order by the same threads with the same
// operations: the result does not depend on how a prompt was cut into steps or on what else is in the batch.
// Sequences are found through device arrays, one block row per sequence the arrays have room for; a row whose
// length is not positive is skipped, so the launches can be recorded.
//
// The scan's block is eight warps on one head's state, 16 value columns of it: warps 0-3 compute (16 columns x 8
// lanes over the key channels, a lane keeping NPL of them in registers), warps 4-7 load the next chunk of tokens
// (r, k, the decay, the bonus sum, v) into the other half of shared memory meanwhile.
#include "common.cuh"

#include <math.h>

#include <type_traits>

namespace {

#define WKV_COLS 16
#define WKV_LANES 8

template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ x, const T* __restrict__ carried, const float* __restrict__ mu,
                                       T* __restrict__ out, const int32_t* __restrict__ token_seq, const int32_t* __restrict__ positions,
                                       const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots, int n_tokens, int width,
                                       int n_mix) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= width) return;
    const int seq = token_seq[t];
    if (seq < 0) return;                                   // a padding row
    const int pos = positions[t];
    const float cur = pb_ld(x + (size_t)t * width + c);
    float prev = 0.f;
    if (pos > q_start[seq]) prev = pb_ld(x + (size_t)(t - 1) * width + c);
    else if (pos > 0) prev = pb_ld(carried + (size_t)slots[seq] * width + c);
    const float diff = prev - cur;
    for (int s = 0; s < n_mix; ++s)
        pb_st(out + ((size_t)s * n_tokens + t) * width + c, fmaf(diff, mu[(size_t)s * width + c], cur));
}

template <typename T, int NPL>
__global__ void __launch_bounds__(256)
wkv_scan_kernel(const T* __restrict__ r_in, long long ld_r, const T* __restrict__ k_in, long long ld_k, const T* __restrict__ v_in,
                long long ld_v, const T* __restrict__ w_in, long long ld_w, const float* __restrict__ w0, const float* __restrict__ bonus,
                float* __restrict__ state, float* __restrict__ y, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, int H,
                int D) {
    constexpr int NPAD = NPL * WKV_LANES;
    constexpr int CHUNK = NPL == 32 ? 4 : (NPL == 16 ? 8 : 16);
    constexpr int TOK = 3 * NPAD + WKV_COLS + 4;                  // floats per token: r, k, decay, v, bonus sum (+ padding to 16 bytes)
    constexpr int BUF = CHUNK * TOK;
    __shared__ __align__(16) float sm[2 * BUF];
    pb_grid_dep_launch();
    const int col_blocks = (D + WKV_COLS - 1) / WKV_COLS;
    const int h = blockIdx.x / col_blocks, p_first = (blockIdx.x % col_blocks) * WKV_COLS;
    const int rq = blockIdx.y;
    const int tid = threadIdx.x;
    const bool computes = tid < WKV_COLS * WKV_LANES;
    const int lt = tid - WKV_COLS * WKV_LANES, lw = lt >> 5, lane = tid & 31;
    float w0v[NPL / 4], uv[NPL / 4];                              // of this lane's key channels: written by no kernel, before the wait
#pragma unroll
    for (int i = 0; i < NPL / 4; ++i) {
        const int n = lane + 32 * i;
        w0v[i] = n < D ? w0[(size_t)h * D + n] : 0.f;
        uv[i] = n < D ? bonus[(size_t)h * D + n] : 0.f;
    }
    pb_grid_dep_wait();
    const int first = cu_q[rq], n_tok = cu_q[rq + 1] - first;
    if (n_tok <= 0) return;
    const int n_chunks = (n_tok + CHUNK - 1) / CHUNK;

    const int colp = tid / WKV_LANES, j = tid % WKV_LANES;
    const int p = p_first + colp;
    const bool live = computes && p < D;
    const int pp = p < D ? p : D - 1;
    float* S = state + (((size_t)slots[rq] * H + h) * D) * D + pp;
    float s[NPL];
    if (computes) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) { const int n = ((i >> 2) * WKV_LANES + j) * 4 + (i & 3); s[i] = n < D ? S[(size_t)n * D] : 0.f; }
    }
    if (D < NPAD) {
        if (!computes)
            for (int idx = lt; idx < 2 * BUF; idx += 128) sm[idx] = 0.f;
        __syncthreads();
    }
    // A loading warp has CHUNK / 4 tokens of a chunk: it asks for all their rows before it works on the first, so the
    // trips to memory overlap (a token past the chunk's end repeats the last one's addresses and is dropped).  A chunk of
    // at most four tokens, a decode step's, is one token a warp.
    auto load_tokens = [&](int k, auto per_warp) {
        constexpr int TPW = decltype(per_warp)::value;
        float* buf = sm + (k & 1) * BUF;
        const int t0 = k * CHUNK, cnt = min(CHUNK, n_tok - t0);
        float rv[TPW][NPL / 4], kv[TPW][NPL / 4], wv[TPW][NPL / 4], vv[TPW];
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
            const int tt = lw + 4 * u;
            const size_t t = (size_t)(first + t0 + min(tt, cnt - 1));
            const T* rr = r_in + t * ld_r + (size_t)h * D;
            const T* kr = k_in + t * ld_k + (size_t)h * D;
            const T* wr = w_in + t * ld_w + (size_t)h * D;
#pragma unroll
            for (int i = 0; i < NPL / 4; ++i) {
                const int n = lane + 32 * i;
                rv[u][i] = n < D ? pb_ld(rr + n) : 0.f;
                kv[u][i] = n < D ? pb_ld(kr + n) : 0.f;
                wv[u][i] = n < D ? pb_ld(wr + n) : 0.f;
            }
            vv[u] = (lane < WKV_COLS && p_first + lane < D) ? pb_ld(v_in + t * ld_v + (size_t)h * D + p_first + lane) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
            const int tt = lw + 4 * u;
            if (tt >= cnt) break;
            float ruk = 0.f;
            float* dst = buf + tt * TOK;
#pragma unroll
            for (int i = 0; i < NPL / 4; ++i) {
                const int n = lane + 32 * i;
                ruk = fmaf(rv[u][i] * uv[i], kv[u][i], ruk);
                if (n < D) { dst[n] = rv[u][i]; dst[NPAD + n] = kv[u][i]; dst[2 * NPAD + n] = expf(-expf(wv[u][i] + w0v[i])); }
            }
            ruk = pb_warp_sum(ruk);
            if (lane < WKV_COLS) dst[3 * NPAD + lane] = vv[u];
            if (lane == 0) dst[3 * NPAD + WKV_COLS] = ruk;
        }
    };
    auto load_chunk = [&](int k) {
        if (n_tok - k * CHUNK <= 4) load_tokens(k, std::integral_constant<int, 1>{});
        else load_tokens(k, std::integral_constant<int, CHUNK / 4>{});
    };
    if (!computes) load_chunk(0);
    __syncthreads();
    for (int k = 0; k < n_chunks; ++k) {
        if (!computes) {
            if (k + 1 < n_chunks) load_chunk(k + 1);
        } else {
            const float* buf = sm + (k & 1) * BUF;
            const int t0 = k * CHUNK, cnt = min(CHUNK, n_tok - t0);
            for (int tt = 0; tt < cnt; ++tt) {
                const float* tok = buf + tt * TOK;
                const float4* r4 = reinterpret_cast<const float4*>(tok) + j;
                const float4* k4 = reinterpret_cast<const float4*>(tok + NPAD) + j;
                const float4* w4 = reinterpret_cast<const float4*>(tok + 2 * NPAD) + j;
                const float v = tok[3 * NPAD + colp], ruk = tok[3 * NPAD + WKV_COLS];
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;    // four sums side by side, added up in a fixed order
#pragma unroll
                for (int i = 0; i < NPL / 4; ++i) {
                    const float4 rr = r4[i * WKV_LANES], kk = k4[i * WKV_LANES], ww = w4[i * WKV_LANES];
                    a0 = fmaf(s[4 * i + 0], rr.x, a0); s[4 * i + 0] = fmaf(ww.x, s[4 * i + 0], kk.x * v);
                    a1 = fmaf(s[4 * i + 1], rr.y, a1); s[4 * i + 1] = fmaf(ww.y, s[4 * i + 1], kk.y * v);
                    a2 = fmaf(s[4 * i + 2], rr.z, a2); s[4 * i + 2] = fmaf(ww.z, s[4 * i + 2], kk.z * v);
                    a3 = fmaf(s[4 * i + 3], rr.w, a3); s[4 * i + 3] = fmaf(ww.w, s[4 * i + 3], kk.w * v);
                }
                float o = (a0 + a1) + (a2 + a3);                 // own channels, then the 8 lanes by three exchanges
                o += __shfl_xor_sync(0xffffffffu, o, 1);
                o += __shfl_xor_sync(0xffffffffu, o, 2);
                o += __shfl_xor_sync(0xffffffffu, o, 4);
                if (live && j == 0) y[(size_t)(first + t0 + tt) * ((size_t)H * D) + (size_t)h * D + p] = fmaf(ruk, v, o);
            }
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) { const int n = ((i >> 2) * WKV_LANES + j) * 4 + (i & 3); if (n < D) S[(size_t)n * D] = s[i]; }
    }
}

}  // namespace

// x [n_tokens, width] dense; carried [slots, width] of x's type; mu float32 [n_mix, width]; out [n_mix, n_tokens, width].
PB_API int pb_token_shift_mix(const void* x, const void* carried, const float* mu, void* out, int dtype, const int32_t* token_seq,
                              const int32_t* positions, const int32_t* q_start, const int32_t* slots, int n_tokens, int width, int n_mix,
                              cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && width > 0 && n_mix > 0, "token_shift_mix: bad sizes");
    PB_REQUIRE(x && carried && mu && out && token_seq && positions && q_start && slots, "token_shift_mix: null pointer");
    if (n_tokens == 0) return 0;
    PB_REQUIRE((width + 127) / 128 < 65536, "token_shift_mix: rows of %d", width);
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(token_shift_mix_kernel<T>, dim3(n_tokens, (width + 127) / 128), dim3(128), 0, stream, (const T*)x, (const T*)carried, mu,
                   (T*)out, token_seq, positions, q_start, slots, n_tokens, width, n_mix)));
    PB_CHECK_LAUNCH("token_shift_mix");
    return 0;
}

// r_in, k_in, v_in, w_in: [n_tokens, H * D] views with dense rows (ld_* apart); w0, bonus float32 [H * D]; state float32
// [slots, H, D, D] (key channel, value); y float32 [n_tokens, H * D] dense.  cu_q [n_seqs + 1], slots [n_seqs].
PB_API int pb_wkv_scan(const void* r_in, long long ld_r, const void* k_in, long long ld_k, const void* v_in, long long ld_v, const void* w_in,
                       long long ld_w, int dtype, const float* w0, const float* bonus, float* state, float* y, const int32_t* cu_q,
                       const int32_t* slots, int n_seqs, int H, int D, cudaStream_t stream) {
    PB_REQUIRE(n_seqs >= 0 && H > 0 && D > 0, "wkv_scan: bad sizes");
    PB_REQUIRE(D <= 32 * WKV_LANES, "wkv_scan: heads of %d elements (at most %d)", D, 32 * WKV_LANES);
    PB_REQUIRE(r_in && k_in && v_in && w_in && w0 && bonus && state && y && cu_q && slots, "wkv_scan: null pointer");
    const long long cols = (long long)H * D;
    PB_REQUIRE(ld_r >= cols && ld_k >= cols && ld_v >= cols && ld_w >= cols, "wkv_scan: rows too short");
    if (n_seqs == 0) return 0;
    PB_REQUIRE(n_seqs < 65536, "wkv_scan: %d sequences in one launch", n_seqs);
    const int col_blocks = (D + WKV_COLS - 1) / WKV_COLS;
    const dim3 grid(H * col_blocks, n_seqs), block(2 * WKV_COLS * WKV_LANES);
    const int npl = (D + WKV_LANES - 1) / WKV_LANES;
#define WKV_LAUNCH(NPL)                                                                                                           \
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(wkv_scan_kernel<T, NPL>, grid, block, 0, stream, (const T*)r_in, ld_r, (const T*)k_in, ld_k,      \
                                           (const T*)v_in, ld_v, (const T*)w_in, ld_w, w0, bonus, state, y, cu_q, slots, H, D)))
    if (npl <= 4) WKV_LAUNCH(4);
    else if (npl <= 8) WKV_LAUNCH(8);
    else if (npl <= 16) WKV_LAUNCH(16);
    else WKV_LAUNCH(32);
#undef WKV_LAUNCH
    PB_CHECK_LAUNCH("wkv_scan");
    return 0;
}
