// Routed experts: the router's choice, the grouping of a step's (token, choice) pairs by expert, the experts'
// products over those groups, and the weighted sum of a token's choices.  Nothing here decides on the host:
// counts, offsets and the map from tiles to experts stay on the device, so a step through a mixture of experts
// has the shape of its token count alone and can be recorded.
//
//   route    scores s = sigmoid(z) of float32 router logits; experts form `groups` equal runs of neighbours, a
//            group's score is the sum of its `gtop` largest scores, only experts of the `keep` best groups can
//            be chosen; the `top` largest allowed scores are chosen (ties: the smaller index), their weights are
//            the scores themselves (or, with `renorm`, divided by their sum).  With a `correction` per expert the
//            choice (group scores and the chosen experts) goes by s + correction, which may be negative; the
//            weights stay the scores s without it.
//   sort     slot i = token * top + choice.  The slots are grouped by expert: offsets[e] .. offsets[e + 1] are the
//            places of expert e, order[place] = slot, place_of[slot] = place, and the places are cut into row
//            tiles of MOE_BM that never span two experts (tile_expert, tile_row0; -1 behind the last tile).
//   products h[place] = silu(Wg_e x) * (Wu_e x) with x the row of slot / top, then y[place] = Wd_e h[place].
//            An output element is summed over k in ascending order by one thread (float32 units) or one
//            tensor-core accumulator (bfloat16), whatever its place in the tile, so a token's result does not
//            depend on who else chose the expert.
//   combine  out[t] = sum over choices c, in order, of w[t, c] * y[place_of[t * top + c]], in float32.
#include "common.cuh"

#include <math.h>
#include <mma.h>

#define MOE_BM 64
#define MOE_BM_LARGE 128
#define MOE_BN 64
#define MOE_BK 16
#define MOE_MAX_TOP 32
#define MOE_MAX_GROUPS 64
#define MOE_MAX_GTOP 8
#define MOE_MAX_EXPERTS 1024

// 16 bytes of a row as floats: 4 of float32, 8 of bfloat16
__device__ __forceinline__ void pb_ld16(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void pb_ld16(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}

// Router logits in 32-bit: out[t, e] = sum_k x[t, k] * W[e, k], every product exact in float32 (the operands are
// float32, or bfloat16 whose products fit), float32 sums.  A warp takes a token and four experts; a lane sums every
// 32nd element in ascending order and the lanes meet in a fixed tree, so the order depends on K alone.
template <typename T>
__global__ void __launch_bounds__(128) router_logits_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ W,
                                                            float* __restrict__ out, int n_tokens, int n_experts, int K) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int lane = threadIdx.x & 31;
    const int per_token = (n_experts + 3) / 4;
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * per_token) return;
    const int t = (int)(item / per_token), e0 = (int)(item % per_token) * 4;
    const T* xr = x + (size_t)t * ldx;
    const T* w0 = W + (size_t)e0 * K;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int k = lane; k < K; k += 32) {
        const float xv = pb_ld(xr + k);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (e0 + j < n_experts) acc[j] = fmaf(xv, pb_ld(w0 + (size_t)j * K + k), acc[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float v = pb_warp_sum(acc[j]);
        if (lane == 0 && e0 + j < n_experts) out[(size_t)t * n_experts + e0 + j] = v;
    }
}

// The same with 16 bytes per load: a lane takes runs of 16 bytes, every 32nd run, in ascending order, its elements one
// after the other; the order of the sums still depends on K alone.  K a multiple of the run, rows 16-byte aligned.
template <typename T>
__global__ void __launch_bounds__(128) router_logits_vec_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ W,
                                                                float* __restrict__ out, int n_tokens, int n_experts, int K) {
    constexpr int VN = 16 / sizeof(T);
    pb_grid_dep_launch();
    const int lane = threadIdx.x & 31;
    const int per_token = (n_experts + 3) / 4;
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * per_token) return;
    const int t = (int)(item / per_token), e0 = (int)(item % per_token) * 4;
    const T* xr = x + (size_t)t * ldx;
    const T* w0 = W + (size_t)e0 * K;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    pb_grid_dep_wait();
#pragma unroll 2
    for (int k = lane * VN; k < K; k += 32 * VN) {
        float xv[VN], wv[4][VN];
        pb_ld16(xr + k, xv);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (e0 + j < n_experts) pb_ld16(w0 + (size_t)j * K + k, wv[j]);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (e0 + j < n_experts) {
#pragma unroll
                for (int e = 0; e < VN; ++e) acc[j] = fmaf(xv[e], wv[j][e], acc[j]);
            }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float v = pb_warp_sum(acc[j]);
        if (lane == 0 && e0 + j < n_experts) out[(size_t)t * n_experts + e0 + j] = v;
    }
}

PB_API int pb_router_logits(const void* x, long long ldx, const void* W, float* out, int dtype, int n_tokens, int n_experts, int K,
                            cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && n_experts > 0 && K > 0 && ldx >= K, "router_logits: bad sizes T=%d E=%d K=%d", n_tokens, n_experts, K);
    PB_REQUIRE(x && W && out, "router_logits: null pointer");
    if (n_tokens == 0) return 0;
    const long long items = (long long)n_tokens * ((n_experts + 3) / 4);
    PB_REQUIRE((items + 3) / 4 < (1ll << 31), "router_logits: too many rows");
    const int vn = dtype == PB_BF16 ? 8 : 4;
    if (K % vn == 0 && ldx % vn == 0 && pb_aligned(x, 16) && pb_aligned(W, 16)) {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(router_logits_vec_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const T*)x, ldx, (const T*)W,
                       out, n_tokens, n_experts, K)));
        PB_CHECK_LAUNCH("router_logits");
        return 0;
    }
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(router_logits_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const T*)x, ldx, (const T*)W, out,
                   n_tokens, n_experts, K)));
    PB_CHECK_LAUNCH("router_logits");
    return 0;
}

// One warp per token.  Lane l holds the scores of experts l, l + 32, ...; a choice is a warp-wide argmax (larger
// score, then smaller index), so a token costs (groups * gtop + top) rounds of five shuffles instead of as many
// passes of one thread over all experts.
__device__ __forceinline__ void moe_warp_argmax(float& val, int& idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, val, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > val || (ov == val && oi < idx)) { val = ov; idx = oi; }
    }
}

template <int SLOTS>                                         // experts per lane: n_experts <= 32 * SLOTS
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ correction,
                                                        int n_tokens, int n_experts, int top, int groups, int keep, int gtop,
                                                        int renorm, int32_t* __restrict__ ids, float* __restrict__ weights) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const float* z = logits + (size_t)t * n_experts;
    const int per = n_experts / groups;
    constexpr int slots = SLOTS;
    const float NONE = -INFINITY;                            // below every choice score, negative ones included
    float sc[SLOTS];                                         // what the choice goes by
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        const int e = lane + 32 * i;
        sc[i] = (i < slots && e < n_experts) ? 1.0f / (1.0f + expf(-z[e])) + (correction ? correction[e] : 0.f) : NONE;
    }
    unsigned long long allowed = groups >= 64 ? ~0ull : ((1ull << groups) - 1ull);
    if (keep < groups) {
        float gscore[MOE_MAX_GROUPS];
        for (int g = 0; g < groups; ++g) {
            unsigned taken = 0u;
            float sum = 0.f;
            const int n = min(gtop, per);
            for (int r = 0; r < n; ++r) {
                float val = NONE;
                int idx = 0x7fffffff;
#pragma unroll
                for (int i = 0; i < SLOTS; ++i) {
                    const int e = lane + 32 * i;
                    if (i < slots && e < n_experts && e / per == g && !((taken >> i) & 1u) && sc[i] > val) { val = sc[i]; idx = e; }
                }
                moe_warp_argmax(val, idx);
                if (idx < n_experts) sum += val;
                if (idx < n_experts && (idx & 31) == lane) taken |= 1u << (idx >> 5);
            }
            gscore[g] = sum;
        }
        allowed = 0ull;
        for (int r = 0; r < keep; ++r) {
            int best = -1;
            for (int g = 0; g < groups; ++g) {
                if ((allowed >> g) & 1ull) continue;
                if (best < 0 || gscore[g] > gscore[best]) best = g;
            }
            allowed |= 1ull << best;
        }
    }
    unsigned chosen = 0u;
    int my_id = 0;
    float my_w = 0.f, total = 0.f;
    for (int r = 0; r < top; ++r) {
        float val = NONE;
        int idx = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) {
            const int e = lane + 32 * i;
            if (i < slots && e < n_experts && ((allowed >> (e / per)) & 1ull) && !((chosen >> i) & 1u) && sc[i] > val) { val = sc[i]; idx = e; }
        }
        moe_warp_argmax(val, idx);
        if (idx >= n_experts) {                              // scores that are no numbers: any allowed expert not yet chosen
            idx = 0;
            val = 0.f;
        } else {
            if ((idx & 31) == lane) chosen |= 1u << (idx >> 5);
            if (correction) val = 1.0f / (1.0f + expf(-z[idx]));          // the weight is the score without the correction
        }
        total += val;
        if (lane == r) { my_id = idx; my_w = val; }
    }
    if (lane < top) {
        ids[(size_t)t * top + lane] = my_id;
        weights[(size_t)t * top + lane] = renorm ? my_w / total : my_w;
    }
}

// correction: float32 [n_experts] added to the scores for the choice only, or null.
PB_API int pb_moe_route(const float* logits, const float* correction, int n_tokens, int n_experts, int top, int groups, int keep,
                        int gtop, int renorm, int32_t* ids, float* weights, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && n_experts > 0 && n_experts <= MOE_MAX_EXPERTS && top > 0 && top <= MOE_MAX_TOP,
               "moe_route: bad sizes T=%d E=%d top=%d", n_tokens, n_experts, top);
    PB_REQUIRE(groups > 0 && groups <= MOE_MAX_GROUPS && n_experts % groups == 0 && keep > 0 && keep <= groups && gtop > 0 &&
               gtop <= MOE_MAX_GTOP, "moe_route: %d groups, keep %d, group score over %d", groups, keep, gtop);
    PB_REQUIRE(top <= keep * (n_experts / groups), "moe_route: top=%d experts cannot come from %d groups of %d", top, keep, n_experts / groups);
    PB_REQUIRE(logits && ids && weights, "moe_route: null pointer");
    if (n_tokens == 0) return 0;
    const int per_lane = (n_experts + 31) / 32;
#define ROUTE_LAUNCH(S)                                                                                                          \
    pb_launch(moe_route_kernel<S>, dim3((n_tokens + 3) / 4), dim3(128), 0, stream, logits, correction, n_tokens, n_experts, top, groups, \
              keep, gtop, renorm, ids, weights)
    if (per_lane <= 1) ROUTE_LAUNCH(1);
    else if (per_lane <= 2) ROUTE_LAUNCH(2);
    else if (per_lane <= 4) ROUTE_LAUNCH(4);
    else if (per_lane <= 8) ROUTE_LAUNCH(8);
    else ROUTE_LAUNCH(32);
#undef ROUTE_LAUNCH
    PB_CHECK_LAUNCH("moe_route");
    return 0;
}

// One block.  ids [n_slots] in [0, n_experts); offsets [n_experts + 1]; order, place_of [n_slots];
// tile_expert, tile_row0 [max_tiles], max_tiles >= ceil(n_slots / MOE_BM) + n_experts.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int32_t* __restrict__ ids, int n_slots, int n_experts,
                                                        int32_t* __restrict__ offsets, int32_t* __restrict__ order,
                                                        int32_t* __restrict__ place_of, int32_t* __restrict__ tile_expert,
                                                        int32_t* __restrict__ tile_row0, int max_tiles, int tile_rows) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ int count[MOE_MAX_EXPERTS], start[MOE_MAX_EXPERTS + 1], tile0[MOE_MAX_EXPERTS + 1];
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
        const int e = min(max(ids[i], 0), n_experts - 1);
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < n_experts; ++e) {
            start[e] = at;
            tile0[e] = tiles;
            at += count[e];
            tiles += (count[e] + tile_rows - 1) / tile_rows;
        }
        start[n_experts] = at;
        tile0[n_experts] = tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) offsets[e] = start[e];
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        for (int k = 0, n = tile0[e + 1] - tile0[e]; k < n; ++k) {
            if (tile0[e] + k < max_tiles) {
                tile_expert[tile0[e] + k] = e;
                tile_row0[tile0[e] + k] = start[e] + k * tile_rows;
            }
        }
        count[e] = 0;                                       // now the cursor of the expert's places
    }
    for (int i = tile0[n_experts] + threadIdx.x; i < max_tiles; i += blockDim.x) {
        tile_expert[i] = -1;
        tile_row0[i] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
        const int e = min(max(ids[i], 0), n_experts - 1);
        const int place = start[e] + atomicAdd(&count[e], 1);
        order[place] = i;
        place_of[i] = place;
    }
}

// Rows of a tile: 128 where the experts have many rows each (prompt steps: the large-tile kernel), else 64.
PB_API int pb_moe_tile_rows(int n_slots, int n_experts) { return n_slots >= 48 * n_experts ? MOE_BM_LARGE : MOE_BM; }

PB_API int pb_moe_sort(const int32_t* ids, int n_slots, int n_experts, int32_t* offsets, int32_t* order, int32_t* place_of,
                       int32_t* tile_expert, int32_t* tile_row0, int max_tiles, int tile_rows, cudaStream_t stream) {
    PB_REQUIRE(n_slots >= 0 && n_experts > 0 && n_experts <= MOE_MAX_EXPERTS, "moe_sort: bad sizes slots=%d E=%d", n_slots, n_experts);
    PB_REQUIRE(tile_rows == MOE_BM || tile_rows == MOE_BM_LARGE || tile_rows == 256, "moe_sort: tiles have %d, %d or 256 rows", MOE_BM, MOE_BM_LARGE);
    PB_REQUIRE(max_tiles >= (n_slots + tile_rows - 1) / tile_rows + n_experts, "moe_sort: room for %d tiles is too little", max_tiles);
    PB_REQUIRE(ids && offsets && order && place_of && tile_expert && tile_row0, "moe_sort: null pointer");
    pb_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, ids, n_slots, n_experts, offsets, order, place_of, tile_expert,
              tile_row0, max_tiles, tile_rows);
    PB_CHECK_LAUNCH("moe_sort");
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// The experts' products on the float32 units (the 32-bit path; also bfloat16 storage with float32 arithmetic).
// C[place, n] = sum_k A[src(place), k] * W_e[n, k]; gated: silu(sum with gate rows) * (sum with up rows), the
// expert's weight being [2 N, K], gate rows first.  src(place) = order[place] / a_div when `order` is given (the
// token of a slot), else the place itself.
// ---------------------------------------------------------------------------------------------------------------
template <typename T, typename TC, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_fma_kernel(const T* __restrict__ A, long long lda, const int32_t* __restrict__ order,
                                                           int a_div, const T* __restrict__ W, long long w_expert_stride, int N,
                                                           int K, const int32_t* __restrict__ tile_expert,
                                                           const int32_t* __restrict__ tile_row0,
                                                           const int32_t* __restrict__ offsets, TC* __restrict__ C, long long ldc) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int row0 = tile_row0[blockIdx.x], row_end = offsets[e + 1];
    const int n0 = blockIdx.y * MOE_BN;
    __shared__ float As[MOE_BK][MOE_BM + 1];
    __shared__ float Ws[GATED ? 2 : 1][MOE_BK][MOE_BN + 1];
    __shared__ int src_s[MOE_BM];
    const int tid = threadIdx.x;
    if (tid < MOE_BM) {
        const int p = row0 + tid;
        src_s[tid] = p < row_end ? (order ? order[p] / a_div : p) : -1;
    }
    __syncthreads();
    const int tx = tid % 16, ty = tid / 16;
    const T* We = W + (size_t)e * w_expert_stride;
    float acc[GATED ? 2 : 1][4][4];
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * 256;
            const int row = idx / MOE_BK, kk = idx % MOE_BK;
            const int gk = k0 + kk, gn = n0 + row;
            const int src = src_s[row];
            As[kk][row] = (src >= 0 && gk < K) ? pb_ld(A + (size_t)src * lda + gk) : 0.f;
            Ws[0][kk][row] = (gn < N && gk < K) ? pb_ld(We + (size_t)gn * K + gk) : 0.f;
            if (GATED) Ws[GATED ? 1 : 0][kk][row] = (gn < N && gk < K) ? pb_ld(We + (size_t)(N + gn) * K + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float a[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g) {
                float b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Ws[g][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(a[i], b[j], acc[g][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = row0 + ty * 4 + i;
        if (p >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[0][i][j];
            if (GATED) v = v / (1.0f + expf(-v)) * acc[GATED ? 1 : 0][i][j];
            pb_st(C + (size_t)p * ldc + gn, v);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same products on the tensor cores: bfloat16 operands, float32 accumulators (mma.sync m16n8k16 through the
// warp-matrix interface), 64 x 64 tiles, eight warps each owning a 16 x 32 piece (gated: of both products).
// Rows of A are gathered through `order`; K in steps of 32 with 16-byte loads.  Needs K % 8 == 0.
// ---------------------------------------------------------------------------------------------------------------
#define MOE_TK 32
#define MOE_LD (MOE_TK + 8)

template <typename TC, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_bf16_kernel(const __nv_bfloat16* __restrict__ A, long long lda,
                                                            const int32_t* __restrict__ order, int a_div,
                                                            const __nv_bfloat16* __restrict__ W, long long w_expert_stride, int N,
                                                            int K, const int32_t* __restrict__ tile_expert,
                                                            const int32_t* __restrict__ tile_row0,
                                                            const int32_t* __restrict__ offsets, TC* __restrict__ C, long long ldc) {
    using namespace nvcuda;
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int row0 = tile_row0[blockIdx.x], row_end = offsets[e + 1];
    const int n0 = blockIdx.y * MOE_BN;
    __shared__ __align__(32) __nv_bfloat16 As[MOE_BM][MOE_LD];
    __shared__ __align__(32) __nv_bfloat16 Ws[GATED ? 2 : 1][MOE_BN][MOE_LD];
    __shared__ __align__(32) float Cs[8][16][36];
    __shared__ int src_s[MOE_BM];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < MOE_BM) {
        const int p = row0 + tid;
        src_s[tid] = p < row_end ? (order ? order[p] / a_div : p) : -1;
    }
    __syncthreads();
    const __nv_bfloat16* We = W + (size_t)e * w_expert_stride;
    const int wm = warp / 2, wn = warp % 2;                  // the warp's piece: rows 16 wm .., columns 32 wn ..
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[GATED ? 2 : 1][2];
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[g][j], 0.f);
    const int lr = tid / 4, lc = (tid % 4) * 8;               // this thread's 16-byte piece of a 64 x 32 tile
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        const bool kin = k0 + lc < K;
        const int src = src_s[lr];
        *reinterpret_cast<uint4*>(&As[lr][lc]) = (src >= 0 && kin) ? *reinterpret_cast<const uint4*>(A + (size_t)src * lda + k0 + lc) : zero;
        const int gn = n0 + lr;
        *reinterpret_cast<uint4*>(&Ws[0][lr][lc]) = (gn < N && kin) ? *reinterpret_cast<const uint4*>(We + (size_t)gn * K + k0 + lc) : zero;
        if (GATED)
            *reinterpret_cast<uint4*>(&Ws[GATED ? 1 : 0][lr][lc]) =
                (gn < N && kin) ? *reinterpret_cast<const uint4*>(We + (size_t)(N + gn) * K + k0 + lc) : zero;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
            wmma::load_matrix_sync(a, &As[wm * 16][kk], MOE_LD);
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> b;
                    wmma::load_matrix_sync(b, &Ws[g][wn * 32 + j * 16][kk], MOE_LD);
                    wmma::mma_sync(acc[g][j], a, b, acc[g][j]);
                }
        }
        __syncthreads();
    }
    if (GATED) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < acc[0][j].num_elements; ++i) {
                const float v = acc[0][j].x[i];
                acc[0][j].x[i] = v / (1.0f + expf(-v)) * acc[GATED ? 1 : 0][j].x[i];
            }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) wmma::store_matrix_sync(&Cs[warp][0][j * 16], acc[0][j], 36, wmma::mem_row_major);
    __syncwarp();
    for (int i = lane; i < 16 * 32; i += 32) {
        const int r = i / 32, c = i % 32;
        const int p = row0 + wm * 16 + r, gn = n0 + wn * 32 + c;
        if (p < row_end && gn < N) pb_st(C + (size_t)p * ldc + gn, Cs[warp][r][c]);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The products of prompt steps, where an expert has rows by the hundred: tiles of 128 rows x 128 weight rows (gated:
// 64 gate rows and the 64 up rows of the same features), K in steps of 64 through a three-stage ring of asynchronous
// 16-byte copies, eight warps of 64 x 32 each (gated: 16 gate and the matching 16 up columns, so that a thread holds
// both factors of its outputs), operands by ldmatrix, mma.sync m16n8k16.  Needs K % 8 == 0.
// ---------------------------------------------------------------------------------------------------------------
#define MOE_LK 64
#define MOE_LS (MOE_LK + 8)
#define MOE_LSTAGES 3
#define MOE_LARGE_SMEM (MOE_LSTAGES * 2 * 128 * MOE_LS * 2)

__device__ __forceinline__ void moe_cp16(void* smem, const void* gmem, bool pred) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    int n = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(sa), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void moe_ldsm4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void moe_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TC, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_large_kernel(const __nv_bfloat16* __restrict__ A, long long lda,
                                                             const int32_t* __restrict__ order, int a_div,
                                                             const __nv_bfloat16* __restrict__ W, long long w_expert_stride, int N,
                                                             int K, const int32_t* __restrict__ tile_expert,
                                                             const int32_t* __restrict__ tile_row0,
                                                             const int32_t* __restrict__ offsets, TC* __restrict__ C, long long ldc) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int row0 = tile_row0[blockIdx.x], row_end = offsets[e + 1];
    constexpr int BN = GATED ? 64 : 128;                      // output columns of a tile
    const int n0 = blockIdx.y * BN;
    extern __shared__ __align__(16) unsigned char moe_smem[];
    __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(moe_smem);                 // [stages][128][MOE_LS]
    __nv_bfloat16* Bs = As + MOE_LSTAGES * 128 * MOE_LS;                             // [stages][128][MOE_LS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, t4 = lane & 3;
    const __nv_bfloat16* We = W + (size_t)e * w_expert_stride;
    // this thread's 16-byte pieces of every 128 x MOE_LK operand tile: piece tid % CPR of rows tid / CPR + n * (256 / CPR)
    constexpr int CPR = MOE_LK / 8, RPP = 256 / CPR, NP = 128 / RPP;
    const int lr = tid / CPR, lc = (tid % CPR) * 8;
    const __nv_bfloat16* a_src[NP];
    const __nv_bfloat16* b_src[NP];
    bool a_ok[NP], b_ok[NP];
#pragma unroll
    for (int n = 0; n < NP; ++n) {
        const int r = lr + RPP * n;
        const int pl = row0 + r;
        const int src = pl < row_end ? (order ? order[pl] / a_div : pl) : -1;
        a_ok[n] = src >= 0;
        a_src[n] = A + (size_t)(src >= 0 ? src : 0) * lda + lc;
        const int col = GATED ? n0 + (r & 63) : n0 + r;
        b_ok[n] = col < N;
        b_src[n] = We + (size_t)((GATED && r >= 64 ? N : 0) + (b_ok[n] ? col : 0)) * K + lc;
    }
    auto load = [&](int st, int k0) {
        const bool kin = k0 + lc < K;
#pragma unroll
        for (int n = 0; n < NP; ++n) {
            moe_cp16(As + ((size_t)st * 128 + lr + RPP * n) * MOE_LS + lc, a_src[n] + k0, a_ok[n] && kin);
            moe_cp16(Bs + ((size_t)st * 128 + lr + RPP * n) * MOE_LS + lc, b_src[n] + k0, b_ok[n] && kin);
        }
    };
    const int wm = warp >> 2, wn = warp & 3;
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    const unsigned sA = (unsigned)__cvta_generic_to_shared(As), sB = (unsigned)__cvta_generic_to_shared(Bs);
    const unsigned a_off = (unsigned)((wm * 64 + (lane & 15)) * MOE_LS + (lane >> 4) * 8) * 2;
    unsigned b_off[2];
#pragma unroll
    for (int nj = 0; nj < 2; ++nj) {
        const int base = GATED ? nj * 64 + wn * 16 : wn * 32 + nj * 16;
        b_off[nj] = (unsigned)((base + (lane >> 4) * 8 + (lane & 7)) * MOE_LS + ((lane >> 3) & 1) * 8) * 2;
    }
    const int KT = (K + MOE_LK - 1) / MOE_LK;
#pragma unroll
    for (int s0 = 0; s0 < MOE_LSTAGES - 1; ++s0) {
        if (s0 < KT) load(s0, s0 * MOE_LK);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int kt = 0; kt < KT; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(MOE_LSTAGES - 2));
        __syncthreads();
        if (kt + MOE_LSTAGES - 1 < KT) load((kt + MOE_LSTAGES - 1) % MOE_LSTAGES, (kt + MOE_LSTAGES - 1) * MOE_LK);
        asm volatile("cp.async.commit_group;\n" ::);
        const unsigned stA = sA + (unsigned)((kt % MOE_LSTAGES) * 128 * MOE_LS * 2), stB = sB + (unsigned)((kt % MOE_LSTAGES) * 128 * MOE_LS * 2);
#pragma unroll
        for (int kk = 0; kk < MOE_LK / 16; ++kk) {
            unsigned a[4][4], b[2][4];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) moe_ldsm4(a[mi], stA + a_off + (unsigned)(mi * 16 * MOE_LS * 2) + kk * 32);
#pragma unroll
            for (int nj = 0; nj < 2; ++nj) moe_ldsm4(b[nj], stB + b_off[nj] + kk * 32);
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) moe_mma(acc[mi][nt], a[mi], b[nt >> 1][(nt & 1) * 2], b[nt >> 1][(nt & 1) * 2 + 1]);
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int pl = row0 + wm * 64 + mi * 16 + gid + 8 * h;
            if (pl >= row_end) continue;
            TC* crow = C + (size_t)pl * ldc;
#pragma unroll
            for (int nt = 0; nt < (GATED ? 2 : 4); ++nt) {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int col = n0 + (GATED ? wn * 16 : wn * 32) + nt * 8 + 2 * t4 + q;
                    if (col >= N) continue;
                    float v = acc[mi][nt][2 * h + q];
                    if (GATED) v = v / (1.0f + expf(-v)) * acc[mi][nt + (GATED ? 2 : 0)][2 * h + q];
                    pb_st(crow + col, v);
                }
            }
        }
    }
}

// A [*, K] with row stride lda; order null or int32 [places]; W [E, (2) N, K] dense, w_expert_stride elements from one
// expert to the next; C [places, N] with row stride ldc, of type out_dtype (float32 or the input's).  grid: max_tiles.
PB_API int pb_moe_gemm(const void* A, long long lda, const int32_t* order, int a_div, const void* W, long long w_expert_stride,
                       int N, int K, int gated, const int32_t* tile_expert, const int32_t* tile_row0, const int32_t* offsets,
                       int max_tiles, int tile_rows, void* C, long long ldc, int dtype, int out_dtype, cudaStream_t stream) {
    PB_REQUIRE(tile_rows == MOE_BM || tile_rows == MOE_BM_LARGE, "moe_gemm: tiles have %d or %d rows", MOE_BM, MOE_BM_LARGE);
    PB_REQUIRE(N > 0 && K > 0 && max_tiles >= 0 && a_div > 0, "moe_gemm: bad sizes N=%d K=%d", N, K);
    PB_REQUIRE(lda >= K && ldc >= N && w_expert_stride >= (long long)(gated ? 2 : 1) * N * K, "moe_gemm: a stride is shorter than its row");
    PB_REQUIRE(A && W && C && tile_expert && tile_row0 && offsets, "moe_gemm: null pointer");
    PB_REQUIRE(out_dtype == PB_F32 || out_dtype == dtype, "moe_gemm: output is float32 or of the input's type");
    if (max_tiles == 0) return 0;
    dim3 grid(max_tiles, (N + MOE_BN - 1) / MOE_BN);
    PB_REQUIRE(grid.y < 65536, "moe_gemm: N=%d too large", N);
#define MOE_LAUNCH(KERNEL, TA, TCC, G)                                                                                         \
    pb_launch(KERNEL, grid, dim3(256), 0, stream, (const TA*)A, lda, order, a_div, (const TA*)W, w_expert_stride, N, K, tile_expert, \
              tile_row0, offsets, (TCC*)C, ldc)
    if (dtype == PB_F32) {
        if (gated) MOE_LAUNCH((moe_gemm_fma_kernel<float, float, true>), float, float, 1);
        else MOE_LAUNCH((moe_gemm_fma_kernel<float, float, false>), float, float, 0);
    } else if (dtype == PB_BF16) {
        const bool tc = K % 8 == 0 && lda % 8 == 0 && w_expert_stride % 8 == 0 && pb_aligned(A, 16) && pb_aligned(W, 16);
        PB_REQUIRE(tc || tile_rows == MOE_BM, "moe_gemm: tiles of %d rows need K in multiples of 8 and aligned operands", MOE_BM_LARGE);
        if (tile_rows == MOE_BM_LARGE) {
            grid.y = (N + (gated ? 64 : 128) - 1) / (gated ? 64 : 128);
#define MOE_LARGE(TCC, G)                                                                                                          \
    do {                                                                                                                           \
        static bool set_ = false;                                                                                                  \
        if (!set_) {                                                                                                               \
            cudaFuncSetAttribute(moe_gemm_large_kernel<TCC, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, MOE_LARGE_SMEM);      \
            set_ = true;                                                                                                           \
        }                                                                                                                          \
        pb_launch(moe_gemm_large_kernel<TCC, G>, grid, dim3(256), (size_t)MOE_LARGE_SMEM, stream, (const __nv_bfloat16*)A, lda, order, a_div, \
                  (const __nv_bfloat16*)W, w_expert_stride, N, K, tile_expert, tile_row0, offsets, (TCC*)C, ldc);                  \
    } while (0)
            if (out_dtype == PB_F32) { if (gated) MOE_LARGE(float, true); else MOE_LARGE(float, false); }
            else { if (gated) MOE_LARGE(__nv_bfloat16, true); else MOE_LARGE(__nv_bfloat16, false); }
#undef MOE_LARGE
        } else if (tc) {
            if (out_dtype == PB_F32) {
                if (gated) MOE_LAUNCH((moe_gemm_bf16_kernel<float, true>), __nv_bfloat16, float, 1);
                else MOE_LAUNCH((moe_gemm_bf16_kernel<float, false>), __nv_bfloat16, float, 0);
            } else {
                if (gated) MOE_LAUNCH((moe_gemm_bf16_kernel<__nv_bfloat16, true>), __nv_bfloat16, __nv_bfloat16, 1);
                else MOE_LAUNCH((moe_gemm_bf16_kernel<__nv_bfloat16, false>), __nv_bfloat16, __nv_bfloat16, 0);
            }
        } else {
            if (out_dtype == PB_F32) {
                if (gated) MOE_LAUNCH((moe_gemm_fma_kernel<__nv_bfloat16, float, true>), __nv_bfloat16, float, 1);
                else MOE_LAUNCH((moe_gemm_fma_kernel<__nv_bfloat16, float, false>), __nv_bfloat16, float, 0);
            } else {
                if (gated) MOE_LAUNCH((moe_gemm_fma_kernel<__nv_bfloat16, __nv_bfloat16, true>), __nv_bfloat16, __nv_bfloat16, 1);
                else MOE_LAUNCH((moe_gemm_fma_kernel<__nv_bfloat16, __nv_bfloat16, false>), __nv_bfloat16, __nv_bfloat16, 0);
            }
        }
    } else {
        return pb_fail("moe_gemm: unknown element type code %d", dtype);
    }
#undef MOE_LAUNCH
    PB_CHECK_LAUNCH("moe_gemm");
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// The products of a decode step, where an expert has a row or a few: nothing but the experts' weights to stream.  A
// warp owns two output features (gated: their two gate rows and two up rows), reads those weight rows once in 16-byte
// pieces, 256 elements of K per step, and multiplies them with up to four rows of the tile at a time, which come from
// the first-level cache; float32 sums, lanes met in a fixed tree.  Tiles are the 64-row tiles of the map; an expert
// with more than four rows walks its weights again for the next four.  Needs K % 8 == 0 and 16-byte aligned rows.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void moe_unpack8(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

template <typename TC, bool GATED>
__global__ void __launch_bounds__(256) moe_gemv_kernel(const __nv_bfloat16* __restrict__ A, long long lda,
                                                       const int32_t* __restrict__ order, int a_div,
                                                       const __nv_bfloat16* __restrict__ W, long long w_expert_stride, int N, int K,
                                                       const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ tile_row0,
                                                       const int32_t* __restrict__ offsets, TC* __restrict__ C, long long ldc) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int row0 = tile_row0[blockIdx.x];
    const int rows = min(MOE_BM, offsets[e + 1] - row0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = (blockIdx.y * 8 + warp) * 2;
    if (f0 >= N) return;
    constexpr int NW = GATED ? 4 : 2;
    const __nv_bfloat16* We = W + (size_t)e * w_expert_stride;
    const __nv_bfloat16* wrow[NW];
#pragma unroll
    for (int j = 0; j < NW; ++j) {
        const int f = min(f0 + (j & 1), N - 1);
        wrow[j] = We + (size_t)((GATED && j >= 2 ? N : 0) + f) * K;
    }
    for (int r0 = 0; r0 < rows; r0 += 4) {
        const int R = min(4, rows - r0);
        const __nv_bfloat16* xrow[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int pl = row0 + r0 + min(r, R - 1);
            xrow[r] = A + (size_t)(order ? order[pl] / a_div : pl) * lda;
        }
        float acc[NW][4];
#pragma unroll
        for (int j = 0; j < NW; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll 2
        for (int k = lane * 8; k < K; k += 256) {
            uint4 wv[NW], xv[4];
#pragma unroll
            for (int j = 0; j < NW; ++j) wv[j] = *reinterpret_cast<const uint4*>(wrow[j] + k);
#pragma unroll
            for (int r = 0; r < 4; ++r) xv[r] = *reinterpret_cast<const uint4*>(xrow[r] + k);
            float xf[4][8];
#pragma unroll
            for (int r = 0; r < 4; ++r) moe_unpack8(xv[r], xf[r]);
#pragma unroll
            for (int j = 0; j < NW; ++j) {
                float wf[8];
                moe_unpack8(wv[j], wf);
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j][r] = fmaf(wf[i], xf[r][i], acc[j][r]);
            }
        }
#pragma unroll
        for (int j = 0; j < NW; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[j][r] = pb_warp_sum(acc[j][r]);
        if (lane < 8) {                                      // lane = 2 * row + feature
            const int r = lane >> 1, q = lane & 1;
            if (r < R && f0 + q < N) {
                float v = 0.f, u = 0.f;
#pragma unroll
                for (int rr = 0; rr < 4; ++rr)
#pragma unroll
                    for (int qq = 0; qq < 2; ++qq)
                        if (rr == r && qq == q) { v = acc[qq][rr]; if (GATED) u = acc[GATED ? 2 + qq : qq][rr]; }
                if (GATED) v = v / (1.0f + expf(-v)) * u;
                pb_st(C + (size_t)(row0 + r0 + r) * ldc + f0 + q, v);
            }
        }
    }
}

// As pb_moe_gemm for bfloat16 operands and a map of 64-row tiles, on the streaming kernel above.
PB_API int pb_moe_gemv(const void* A, long long lda, const int32_t* order, int a_div, const void* W, long long w_expert_stride,
                       int N, int K, int gated, const int32_t* tile_expert, const int32_t* tile_row0, const int32_t* offsets,
                       int max_tiles, void* C, long long ldc, int out_dtype, cudaStream_t stream) {
    PB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && w_expert_stride % 8 == 0 && max_tiles >= 0 && a_div > 0,
               "moe_gemv: N=%d K=%d lda=%lld: K and the strides in multiples of 8", N, K, lda);
    PB_REQUIRE(A && W && C && tile_expert && tile_row0 && offsets && pb_aligned(A, 16) && pb_aligned(W, 16), "moe_gemv: null or unaligned pointer");
    PB_REQUIRE(lda >= K && ldc >= N && w_expert_stride >= (long long)(gated ? 2 : 1) * N * K, "moe_gemv: a stride is shorter than its row");
    if (max_tiles == 0) return 0;
    dim3 grid(max_tiles, (N + 15) / 16);
    PB_REQUIRE(grid.y < 65536, "moe_gemv: N=%d too large", N);
#define MOE_GEMV(TCC, G)                                                                                                              \
    pb_launch(moe_gemv_kernel<TCC, G>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)A, lda, order, a_div, (const __nv_bfloat16*)W, \
              w_expert_stride, N, K, tile_expert, tile_row0, offsets, (TCC*)C, ldc)
    if (out_dtype == PB_F32) { if (gated) MOE_GEMV(float, true); else MOE_GEMV(float, false); }
    else if (out_dtype == PB_BF16) { if (gated) MOE_GEMV(__nv_bfloat16, true); else MOE_GEMV(__nv_bfloat16, false); }
    else return pb_fail("moe_gemv: unknown output type code %d", out_dtype);
#undef MOE_GEMV
    PB_CHECK_LAUNCH("moe_gemv");
    return 0;
}

// out[place, :] = x[order[place] / div, :]: the rows of a step's tokens in the order of their places (what a product
// that reads its rows through tensor-map copies needs).
template <typename T>
__global__ void moe_gather_rows_kernel(const T* __restrict__ x, long long ldx, const int32_t* __restrict__ order, int div,
                                       T* __restrict__ out, int width) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const size_t place = blockIdx.x;
    const T* src = x + (size_t)(order[place] / div) * ldx;
    T* dst = out + place * width;
    if (width % (16 / sizeof(T)) == 0 && ldx % (16 / sizeof(T)) == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(out) % 16 == 0) {
        const int n = width / (16 / (int)sizeof(T));
        for (int i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
    }
}

PB_API int pb_moe_gather_rows(const void* x, long long ldx, const int32_t* order, int div, void* out, int dtype, int places,
                              int width, cudaStream_t stream) {
    PB_REQUIRE(places >= 0 && width > 0 && div > 0 && ldx >= width, "moe_gather_rows: bad sizes");
    PB_REQUIRE(x && order && out, "moe_gather_rows: null pointer");
    if (places == 0) return 0;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(moe_gather_rows_kernel<T>, dim3(places), dim3(128), 0, stream, (const T*)x, ldx, order, div, (T*)out, width)));
    PB_CHECK_LAUNCH("moe_gather_rows");
    return 0;
}

// out[t, :] = sum_c w[t, c] * y[place_of[t * top + c], :], choices in ascending order, float32 sums.
template <typename T, typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int32_t* __restrict__ place_of,
                                   const float* __restrict__ weights, T* __restrict__ out, int top, int width) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = 0.f;
        for (int c = 0; c < top; ++c) v = fmaf(weights[t * top + c], pb_ld(y + (size_t)place_of[t * top + c] * width + i), v);
        pb_st(out + t * width + i, v);
    }
}

// y float32 (y_dtype PB_F32) or of the output's type.
PB_API int pb_moe_combine(const void* y, int y_dtype, const int32_t* place_of, const float* weights, void* out, int dtype, int n_tokens,
                          int top, int width, cudaStream_t stream) {
    PB_REQUIRE(y_dtype == PB_F32 || y_dtype == dtype, "moe_combine: y is float32 or of the output's type");
    PB_REQUIRE(n_tokens >= 0 && top > 0 && width > 0, "moe_combine: bad sizes");
    PB_REQUIRE(y && place_of && weights && out, "moe_combine: null pointer");
    if (n_tokens == 0) return 0;
    if (y_dtype == PB_F32) {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(moe_combine_kernel<T, float>, dim3(n_tokens), dim3(width >= 1024 ? 256 : 128), 0, stream, (const float*)y, place_of, weights, (T*)out, top, width)));
    } else {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(moe_combine_kernel<T, T>, dim3(n_tokens), dim3(width >= 1024 ? 256 : 128), 0, stream, (const T*)y, place_of, weights, (T*)out, top, width)));
    }
    PB_CHECK_LAUNCH("moe_combine");
    return 0;
}
