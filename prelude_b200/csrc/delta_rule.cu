// The gated delta rule between its short convolutions and its output norm:
//
//   pb_gated_delta_scan   per head, token by token, with the state S [dim, vdim] in float32:
//                             q <- q / sqrt(sum q^2 + 1e-6) * dim^(-1/2),  k <- k / sqrt(sum k^2 + 1e-6)
//                             beta = sigmoid(b),  g = exp(-exp(A_log) softplus(a + dt_bias))
//                             S <- g S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q
//                         so the read-out sees the current token's write.  Query/key head of head h: h / (heads / kv heads).
//
// Unit norms, sigmoid, softplus, exponentials, the state and every sum over it are float32 whatever the run's type;
// q, k, v (the convolutions' outputs) and the projections b and a are of the run's type.  A sequence's tokens are
// visited in order by the same threads with the same operations, so the result does not depend on how a prompt was
// cut into steps or on what else is in the batch.  The state of a sequence is read at the start of a step from its
// slot and written back at the end.  Sequences are found through device arrays (cumulative lengths, state slots), one
// block row per sequence the arrays have room for; a row whose length is not positive is skipped, so the launch has
// the same shape whatever the step holds and can be recorded.
//
// A block is eight warps on one head's state, 16 columns p of it.  Warps 0-3 compute: 16 columns x 8 lanes over the
// state rows n, a lane keeping NPL rows in registers (rows 4 (8 i + j) .. + 3, so that the lanes of a column read
// consecutive 16-byte pieces of k and q).  Warps 4-7 load: while the others work on one chunk of tokens they put the
// next chunk's unit q and k, its v, beta and g into the other half of shared memory.
#include "common.cuh"

#include <math.h>

#include <type_traits>

namespace {

#define GD_COLS 16
#define GD_LANES 8

__device__ __forceinline__ float gd_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

template <typename T, int NPL>
__global__ void __launch_bounds__(256)
gated_delta_scan_kernel(const T* __restrict__ u_in, long long ld_u, const T* __restrict__ b_in, long long ld_b, const T* __restrict__ a_in,
                        long long ld_a, const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ state,
                        float* __restrict__ y, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, int H, int G, int D,
                        int E) {
    constexpr int NPAD = NPL * GD_LANES;
    constexpr int CHUNK = NPL == 32 ? 8 : 16;
    constexpr int TOK = 2 * NPAD + GD_COLS + 4;                   // floats per token: k, q, v, beta, g (+ padding to 16 bytes)
    constexpr int BUF = CHUNK * TOK;
    __shared__ __align__(16) float sm[2 * BUF];
    pb_grid_dep_launch();
    const int col_blocks = (E + GD_COLS - 1) / GD_COLS;
    const int h = blockIdx.x / col_blocks, p_first = (blockIdx.x % col_blocks) * GD_COLS;
    const int r = blockIdx.y;
    const int tid = threadIdx.x;
    const bool computes = tid < GD_COLS * GD_LANES;
    const float rate = expf(a_log[h]), bias = dt_bias[h];        // written by no kernel: before the wait
    const float q_scale = 1.0f / sqrtf((float)D);
    pb_grid_dep_wait();
    const int first = cu_q[r], n_tok = cu_q[r + 1] - first;
    if (n_tok <= 0) return;
    const int g = h / (H / G);
    const int n_chunks = (n_tok + CHUNK - 1) / CHUNK;

    const int colp = tid / GD_LANES, j = tid % GD_LANES;
    const int p = p_first + colp;
    const bool live = computes && p < E;
    const int pp = p < E ? p : E - 1;                            // idle columns follow along and store nothing
    float* S = state + (((size_t)slots[r] * H + h) * D) * E + pp;
    float s[NPL];
    if (computes) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) { const int n = ((i >> 2) * GD_LANES + j) * 4 + (i & 3); s[i] = n < D ? S[(size_t)n * E] : 0.f; }
    }
    const int lt = tid - GD_COLS * GD_LANES, lw = lt >> 5, lane = tid & 31;
    if (D < NPAD) {                                              // rows past D are read as zeros by the lanes
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
        float qv[TPW][NPL / 4], kv[TPW][NPL / 4], vv[TPW], braw[TPW], araw[TPW];      // NPAD / 32 elements of q and k a lane
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
            const int tt = lw + 4 * u;
            const size_t t = (size_t)(first + t0 + min(tt, cnt - 1));
            const T* row = u_in + t * ld_u;
            const T* qr = row + (size_t)g * D;
            const T* kr = row + (size_t)(G + g) * D;
#pragma unroll
            for (int i = 0; i < NPL / 4; ++i) {
                const int n = lane + 32 * i;
                qv[u][i] = n < D ? pb_ld(qr + n) : 0.f;
                kv[u][i] = n < D ? pb_ld(kr + n) : 0.f;
            }
            vv[u] = (lane < GD_COLS && p_first + lane < E) ? pb_ld(row + (size_t)2 * G * D + (size_t)h * E + p_first + lane) : 0.f;
            braw[u] = araw[u] = 0.f;
            if (lane == 0) { braw[u] = pb_ld(b_in + t * ld_b + h); araw[u] = pb_ld(a_in + t * ld_a + h); }
        }
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
            const int tt = lw + 4 * u;
            if (tt >= cnt) break;
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int i = 0; i < NPL / 4; ++i) {
                sq = fmaf(qv[u][i], qv[u][i], sq);
                sk = fmaf(kv[u][i], kv[u][i], sk);
            }
            const float iq = q_scale / sqrtf(pb_warp_sum(sq) + 1e-6f), ik = 1.0f / sqrtf(pb_warp_sum(sk) + 1e-6f);
            float* dst = buf + tt * TOK;
#pragma unroll
            for (int i = 0; i < NPL / 4; ++i) {
                const int n = lane + 32 * i;
                if (n < D) { dst[n] = kv[u][i] * ik; dst[NPAD + n] = qv[u][i] * iq; }
            }
            if (lane < GD_COLS) dst[2 * NPAD + lane] = vv[u];
            if (lane == 0) {
                dst[2 * NPAD + GD_COLS] = 1.0f / (1.0f + expf(-braw[u]));
                dst[2 * NPAD + GD_COLS + 1] = expf(-rate * gd_softplus(araw[u] + bias));
            }
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
                const float4* k4 = reinterpret_cast<const float4*>(tok) + j;
                const float4* q4 = reinterpret_cast<const float4*>(tok + NPAD) + j;
                const float v = tok[2 * NPAD + colp], beta = tok[2 * NPAD + GD_COLS], decay = tok[2 * NPAD + GD_COLS + 1];
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;    // four sums side by side, added up in a fixed order
#pragma unroll
                for (int i = 0; i < NPL / 4; ++i) {
                    const float4 kk = k4[i * GD_LANES];
                    s[4 * i + 0] *= decay; a0 = fmaf(s[4 * i + 0], kk.x, a0);
                    s[4 * i + 1] *= decay; a1 = fmaf(s[4 * i + 1], kk.y, a1);
                    s[4 * i + 2] *= decay; a2 = fmaf(s[4 * i + 2], kk.z, a2);
                    s[4 * i + 3] *= decay; a3 = fmaf(s[4 * i + 3], kk.w, a3);
                }
                float sk = (a0 + a1) + (a2 + a3);                // (S^T k)[p]: own rows, then the 8 lanes by three exchanges
                sk += __shfl_xor_sync(0xffffffffu, sk, 1);
                sk += __shfl_xor_sync(0xffffffffu, sk, 2);
                sk += __shfl_xor_sync(0xffffffffu, sk, 4);
                const float w = beta * (v - sk);
                a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
                for (int i = 0; i < NPL / 4; ++i) {
                    const float4 kk = k4[i * GD_LANES], qq = q4[i * GD_LANES];
                    s[4 * i + 0] = fmaf(kk.x, w, s[4 * i + 0]); a0 = fmaf(s[4 * i + 0], qq.x, a0);
                    s[4 * i + 1] = fmaf(kk.y, w, s[4 * i + 1]); a1 = fmaf(s[4 * i + 1], qq.y, a1);
                    s[4 * i + 2] = fmaf(kk.z, w, s[4 * i + 2]); a2 = fmaf(s[4 * i + 2], qq.z, a2);
                    s[4 * i + 3] = fmaf(kk.w, w, s[4 * i + 3]); a3 = fmaf(s[4 * i + 3], qq.w, a3);
                }
                float o = (a0 + a1) + (a2 + a3);
                o += __shfl_xor_sync(0xffffffffu, o, 1);
                o += __shfl_xor_sync(0xffffffffu, o, 2);
                o += __shfl_xor_sync(0xffffffffu, o, 4);
                if (live && j == 0) y[(size_t)(first + t0 + tt) * ((size_t)H * E) + (size_t)h * E + p] = o;
            }
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) { const int n = ((i >> 2) * GD_LANES + j) * 4 + (i & 3); if (n < D) S[(size_t)n * E] = s[i]; }
    }
}

}  // namespace

// u: the convolutions' outputs [n_tokens, 2 * G * D + H * E] laid out [q | k | v], rows ld_u apart; b_in, a_in: the
// [n_tokens, H] columns of a projection (rows ld_b, ld_a apart); a_log, dt_bias float32 [H]; state float32
// [slots, H, D, E]; y float32 [n_tokens, H * E] dense.  cu_q [n_seqs + 1], slots [n_seqs].
PB_API int pb_gated_delta_scan(const void* u, long long ld_u, const void* b_in, long long ld_b, const void* a_in, long long ld_a, int dtype,
                               const float* a_log, const float* dt_bias, float* state, float* y, const int32_t* cu_q, const int32_t* slots,
                               int n_seqs, int H, int G, int D, int E, cudaStream_t stream) {
    PB_REQUIRE(n_seqs >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && E > 0, "gated_delta_scan: bad sizes");
    PB_REQUIRE(D <= 32 * GD_LANES, "gated_delta_scan: keys of %d elements (at most %d)", D, 32 * GD_LANES);
    PB_REQUIRE(u && b_in && a_in && a_log && dt_bias && state && y && cu_q && slots, "gated_delta_scan: null pointer");
    PB_REQUIRE(ld_u >= 2ll * G * D + (long long)H * E && ld_b >= H && ld_a >= H, "gated_delta_scan: rows too short");
    if (n_seqs == 0) return 0;
    PB_REQUIRE(n_seqs < 65536, "gated_delta_scan: %d sequences in one launch", n_seqs);
    const int col_blocks = (E + GD_COLS - 1) / GD_COLS;
    const dim3 grid(H * col_blocks, n_seqs), block(2 * GD_COLS * GD_LANES);
    const int npl = (D + GD_LANES - 1) / GD_LANES;
#define GD_LAUNCH(NPL)                                                                                                             \
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(gated_delta_scan_kernel<T, NPL>, grid, block, 0, stream, (const T*)u, ld_u, (const T*)b_in, ld_b, \
                                           (const T*)a_in, ld_a, a_log, dt_bias, state, y, cu_q, slots, H, G, D, E)))
    if (npl <= 4) GD_LAUNCH(4);
    else if (npl <= 8) GD_LAUNCH(8);
    else if (npl <= 16) GD_LAUNCH(16);
    else GD_LAUNCH(32);
#undef GD_LAUNCH
    PB_CHECK_LAUNCH("gated_delta_scan");
    return 0;
}
