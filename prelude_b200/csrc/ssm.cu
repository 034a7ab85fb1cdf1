// A selective state-space mixer with scalar decay per head, between its input and output projections:
//
//   pb_causal_conv_silu     u = silu(conv(xBC) + bias) per channel over the last `taps` tokens; what lies before the
//                           step's first token comes from the sequence's carried inputs
//   pb_conv_state_update    the last taps - 1 inputs of every sequence, carried to its next step
//   pb_ssm_scan             dt = softplus(dt + bias); S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x, token by
//                           token, the state [heads, state, head_dim] float32 per sequence, read at the start and written
//                           at the end of the step
//   pb_decay_scan           the same recurrence with a constant decay per head and no step size: linear attention with a
//                           decaying state, S <- decay S + k v^T; o = S^T q, q, k, v the SiLU of the projection's columns
//   pb_gated_group_rmsnorm  y * silu(z), brought to unit root mean square in equal parts, times a scale; or, with the gate
//                           after the norm, y brought to unit root mean square in equal parts, times a scale, times silu(z)
//
// Decay, step size, softplus, exponentials, the state and the sums over it are float32 whatever the run's type;
// the projections and the convolution's output are of the run's type.  A sequence's tokens are visited in order,
// one after the other, by the same threads: the result does not depend on how a prompt was cut into steps or on
// what else is in the batch.  All kernels find a step's sequences through device arrays (cumulative lengths,
// state slots), with one block row per sequence the arrays have room for: a row whose length is not positive is
// skipped, so the launches have the same shape whatever the step holds and can be recorded.
#include "common.cuh"

#include <math.h>

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ bool pb_aligned_dev(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
// 16 bytes of a row as floats: 4 of float32, 8 of bfloat16
__device__ __forceinline__ void pb_ld_vec(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void pb_ld_vec(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void pb_st_vec(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void pb_st_vec(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, long long ld_in, const float* __restrict__ w,
                                        const float* __restrict__ bias, const T* __restrict__ carried, T* __restrict__ out,
                                        const int32_t* __restrict__ token_seq, const int32_t* __restrict__ positions,
                                        const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots, int n_tokens,
                                        int channels, int taps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= channels) return;
    const int seq = token_seq[t];
    if (seq < 0) return;                                   // a padding row
    const int i = positions[t] - q_start[seq];             // the token's index among its sequence's tokens of this step
    const T* old = carried + (size_t)slots[seq] * (taps - 1) * channels;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int idx = i - (taps - 1 - j);                // in-step index of the input under tap j
        const float x = idx >= 0 ? pb_ld(in + (size_t)(t - (taps - 1 - j)) * ld_in + c)
                                 : pb_ld(old + (size_t)(taps - 1 + idx) * channels + c);
        acc = fmaf(w[(size_t)c * taps + j], x, acc);
    }
    pb_st(out + (size_t)t * channels + c, silu_f(acc));
}

// The same, 16 bytes of channels per thread and a run of consecutive tokens per block (channels, row stride and
// pointers in multiples of 16 bytes; TAPS known at compile time).  A thread keeps its channels' taps and the last
// TAPS - 1 inputs in registers: while the run stays inside one sequence every input is read once.
#define CONV_RUN 16                                          // a long step; a step of few tokens gives every token a block
template <typename T, int TAPS>
__global__ void causal_conv_silu_vec_kernel(const T* __restrict__ in, long long ld_in, const float* __restrict__ w,
                                            const float* __restrict__ bias, const T* __restrict__ carried, T* __restrict__ out,
                                            const int32_t* __restrict__ token_seq, const int32_t* __restrict__ positions,
                                            const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots, int n_tokens,
                                            int channels, int run) {
    constexpr int VN = 16 / sizeof(T);
    pb_grid_dep_launch();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VN;
    if (c >= channels) return;
    float wt[VN][TAPS], bs[VN];
#pragma unroll
    for (int e = 0; e < VN; ++e) {
        bs[e] = bias ? bias[c + e] : 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wt[e][j] = w[(size_t)(c + e) * TAPS + j];
    }
    pb_grid_dep_wait();
    float win[TAPS][VN];                                   // win[j]: the input under tap j
    int prev_seq = -1;
    const int t_end = min(n_tokens, (int)(blockIdx.x + 1) * run);
    for (int t = blockIdx.x * run; t < t_end; ++t) {
        const int seq = token_seq[t];
        if (seq < 0) { prev_seq = -1; continue; }          // a padding row
        const int i = positions[t] - q_start[seq];
        if (seq == prev_seq) {                             // the token after the one before: shift, fetch one
#pragma unroll
            for (int j = 0; j + 1 < TAPS; ++j)
#pragma unroll
                for (int e = 0; e < VN; ++e) win[j][e] = win[j + 1][e];
            pb_ld_vec(in + (size_t)t * ld_in + c, win[TAPS - 1]);
        } else {
            const T* old = carried + (size_t)slots[seq] * (TAPS - 1) * channels;
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                const int idx = i - (TAPS - 1 - j);
                pb_ld_vec(idx >= 0 ? in + (size_t)(t - (TAPS - 1 - j)) * ld_in + c : old + (size_t)(TAPS - 1 + idx) * channels + c, win[j]);
            }
            prev_seq = seq;
        }
        float acc[VN];
#pragma unroll
        for (int e = 0; e < VN; ++e) {
            float a = bs[e];
#pragma unroll
            for (int j = 0; j < TAPS; ++j) a = fmaf(wt[e][j], win[j][e], a);
            acc[e] = silu_f(a);
        }
        pb_st_vec(out + (size_t)t * channels + c, acc);
    }
}

// Row s of a sequence's carried inputs holds the input at in-step index s - (taps - 1) of its NEXT step.  One thread
// owns a (sequence, channel): it reads rows above the one it writes, in ascending order, so nothing is lost.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ in, long long ld_in, T* __restrict__ carried,
                                         const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, int channels, int taps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= channels) return;
    const int first = cu_q[r], n = cu_q[r + 1] - first;
    if (n <= 0) return;
    T* st = carried + (size_t)slots[r] * (taps - 1) * channels;
    for (int s = 0; s < taps - 1; ++s) {
        const int idx = n - (taps - 1) + s;
        st[(size_t)s * channels + c] = idx >= 0 ? in[(size_t)(first + idx) * ld_in + c] : st[(size_t)(taps - 1 + idx) * channels + c];
    }
}

// ---------------------------------------------------------------------------------------------------------
// The scan.  A block is eight warps on one head's state, 16 columns p of it.  Warps 0-3 compute: 16 columns x 8 lanes
// over the state rows n, a lane keeping NPL rows in registers (rows 4 (8 i + j) .. + 3 for i = 0 .. NPL / 4 - 1, so
// that the lanes of a column read consecutive 16-byte pieces of B and C).  Warps 4-7 load: while the others work on
// one chunk of tokens they put the next chunk's x, B, C (as float32), step size dt = softplus(dt + bias) and decay
// exp(-exp(A_log) dt) into the other half of shared memory, so the recurrence, which visits tokens one after the
// other, never waits for global memory.  Per token: S[n][p] = decay S[n][p] + (dt x[p]) B[n],
// y[p] = sum_n S[n][p] C[n] (own rows in ascending order, then the 8 lanes by three exchanges) + D x[p].
#define SCAN_COLS 16
#define SCAN_LANES 8
#ifndef SCAN_UNROLL
#define SCAN_UNROLL 4
#endif

//
// FIXED: the same recurrence with a decay per head that is a constant of the model and no step size (linear attention
// with a decaying state: S <- decay_h S + k v^T, o = S^T q).  x, B, C are then v, k, q read straight from the
// projection's columns (rows `ld_u` apart) and passed through SiLU by the loaders, in float32; dt is 1, D is 0, and
// `a_log` holds the decays themselves.  With `activate` 0 the columns hold SiLU's values already.
template <typename T, int NPL, bool FIXED>
__global__ void __launch_bounds__(256)
ssm_scan_kernel(const T* __restrict__ u, long long ld_u, const T* __restrict__ dt_in, long long ld_dt, const float* __restrict__ dt_bias,
                const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state,
                float* __restrict__ y, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, int heads, int P,
                int N, int groups, int activate) {
    constexpr int NPAD = NPL * SCAN_LANES;                     // state rows with padding: a power of two
    constexpr int CHUNK = NPL == 32 ? 8 : 16;                  // tokens per chunk
    constexpr int BUF = CHUNK * (2 * NPAD + SCAN_COLS + 2);    // floats per half: B, C, x, dt, decay
    __shared__ __align__(16) float sm[2 * BUF];
    pb_grid_dep_launch();
    const int col_blocks = (P + SCAN_COLS - 1) / SCAN_COLS;
    const int h = blockIdx.x / col_blocks, p_first = (blockIdx.x % col_blocks) * SCAN_COLS;
    const int r = blockIdx.y;
    const int tid = threadIdx.x;
    const bool computes = tid < SCAN_COLS * SCAN_LANES;
    // written by no kernel: before the wait
    const float neg_a = FIXED ? a_log[h] : -expf(a_log[h]), bias = FIXED ? 0.f : dt_bias[h], skip = FIXED ? 0.f : d_skip[h];
    pb_grid_dep_wait();
    const int first = cu_q[r], n_tok = cu_q[r + 1] - first;
    if (n_tok <= 0) return;
    const int inner = heads * P, channels = inner + 2 * groups * N;
    const int g = h / (heads / groups);
    const int n_chunks = (n_tok + CHUNK - 1) / CHUNK;

    // compute threads
    const int colp = tid / SCAN_LANES, j = tid % SCAN_LANES;
    const int p = p_first + colp;
    const bool live = computes && p < P;
    const int pp = p < P ? p : P - 1;                                             // idle columns follow along and store nothing
    float* S = state + (((size_t)slots[r] * heads + h) * N) * P + pp;
    float s[NPL];
    if (computes) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) { const int n = ((i >> 2) * SCAN_LANES + j) * 4 + (i & 3); s[i] = n < N ? S[(size_t)n * P] : 0.f; }
    }
    // load threads
    const int lt = tid - SCAN_COLS * SCAN_LANES;
    constexpr int VN = 16 / sizeof(T);                                            // elements of a 16-byte load
    const bool vec = N % VN == 0 && channels % VN == 0 && inner % VN == 0 && ld_u % VN == 0 && pb_aligned_dev(u, 16);
    // every block of a head's columns activates the head's keys and queries anew; a long step has them activated once,
    // in place, by a kernel ahead of this one (`activate` 0)
    auto act = [activate](float v) { return (FIXED && activate) ? silu_f(v) : v; };
    if (N < NPAD) {                                                               // rows past N are read as zeros by the lanes
        if (!computes)
            for (int idx = lt; idx < 2 * BUF; idx += 128) sm[idx] = 0.f;
        __syncthreads();
    }
    auto load_chunk = [&](int k) {
        float* buf = sm + (k & 1) * BUF;
        const int t0 = k * CHUNK, cnt = min(CHUNK, n_tok - t0);
        const T* rows = u + (size_t)(first + t0) * ld_u;
        // everything a thread fetches for the chunk is asked for before anything is stored: one wait per chunk
        float xv[(CHUNK * SCAN_COLS + 127) / 128];
#pragma unroll
        for (int it = 0; it < (CHUNK * SCAN_COLS + 127) / 128; ++it) {
            const int idx = lt + it * 128;
            const int tt = idx / SCAN_COLS, cc = idx % SCAN_COLS;
            xv[it] = (idx < cnt * SCAN_COLS && p_first + cc < P) ? act(pb_ld(rows + (size_t)tt * ld_u + h * P + p_first + cc)) : 0.f;
        }
        const float dt_raw = (!FIXED && lt < cnt) ? pb_ld(dt_in + (size_t)(first + t0 + lt) * ld_dt + h) : 0.f;
        if (vec) {
            // B and C of a token: 2 N / VN pieces of 16 bytes; four of a thread's loads in flight at a time
            const int per_tok = 2 * (N / VN), total = cnt * per_tok;
            for (int base = lt; base < total; base += 4 * 128) {
                float v[4][VN];
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int idx = base + it * 128;
                    if (idx < total) {
                        const int tt = idx / per_tok, rem = idx - tt * per_tok;
                        pb_ld_vec(rows + (size_t)tt * ld_u + inner + g * N + (rem >= N / VN ? (groups - 1) * N : 0) + rem * VN, v[it]);
                    }
                }
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int idx = base + it * 128;
                    if (idx < total) {
                        const int tt = idx / per_tok, rem = idx - tt * per_tok;
                        const bool is_c = rem >= N / VN;
                        float* dst = buf + (is_c ? CHUNK * NPAD : 0) + tt * NPAD + (is_c ? rem - N / VN : rem) * VN;
#pragma unroll
                        for (int e = 0; e < VN; e += 4)
                            *reinterpret_cast<float4*>(dst + e) = make_float4(act(v[it][e]), act(v[it][e + 1]), act(v[it][e + 2]), act(v[it][e + 3]));
                    }
                }
            }
        } else {
            for (int base = lt; base < cnt * N; base += 4 * 128) {
                float vb[4], vc[4];
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int idx = base + it * 128;
                    if (idx < cnt * N) {
                        const int tt = idx / N, n = idx - tt * N;
                        const T* row = rows + (size_t)tt * ld_u + inner + g * N;
                        vb[it] = act(pb_ld(row + n));
                        vc[it] = act(pb_ld(row + groups * N + n));
                    }
                }
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int idx = base + it * 128;
                    if (idx < cnt * N) {
                        const int tt = idx / N, n = idx - tt * N;
                        buf[tt * NPAD + n] = vb[it];
                        buf[CHUNK * NPAD + tt * NPAD + n] = vc[it];
                    }
                }
            }
        }
#pragma unroll
        for (int it = 0; it < (CHUNK * SCAN_COLS + 127) / 128; ++it) {
            const int idx = lt + it * 128;
            if (idx < cnt * SCAN_COLS) buf[2 * CHUNK * NPAD + idx] = xv[it];
        }
        if (!FIXED && lt < cnt) {
            const float dt = softplus_f(dt_raw + bias);
            buf[2 * CHUNK * NPAD + CHUNK * SCAN_COLS + lt] = dt;
            buf[2 * CHUNK * NPAD + CHUNK * SCAN_COLS + CHUNK + lt] = expf(neg_a * dt);
        }
    };
    if (!computes) load_chunk(0);
    __syncthreads();
    for (int k = 0; k < n_chunks; ++k) {
        if (!computes) {
            if (k + 1 < n_chunks) load_chunk(k + 1);
        } else {
            const float* buf = sm + (k & 1) * BUF;
            const int t0 = k * CHUNK, cnt = min(CHUNK, n_tok - t0);
            auto token = [&](int tt) {
                const float x = buf[2 * CHUNK * NPAD + tt * SCAN_COLS + colp];
                const float dt = FIXED ? 1.0f : buf[2 * CHUNK * NPAD + CHUNK * SCAN_COLS + tt];
                const float decay = FIXED ? neg_a : buf[2 * CHUNK * NPAD + CHUNK * SCAN_COLS + CHUNK + tt];
                const float dx = FIXED ? x : dt * x;
                const float4* b4 = reinterpret_cast<const float4*>(buf + tt * NPAD) + j;
                const float4* c4 = reinterpret_cast<const float4*>(buf + CHUNK * NPAD + tt * NPAD) + j;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;                   // four sums side by side, added up in a fixed order
#pragma unroll
                for (int i = 0; i < NPL / 4; ++i) {
                    const float4 b = b4[i * SCAN_LANES], c = c4[i * SCAN_LANES];
                    s[4 * i + 0] = fmaf(decay, s[4 * i + 0], dx * b.x); a0 = fmaf(s[4 * i + 0], c.x, a0);
                    s[4 * i + 1] = fmaf(decay, s[4 * i + 1], dx * b.y); a1 = fmaf(s[4 * i + 1], c.y, a1);
                    s[4 * i + 2] = fmaf(decay, s[4 * i + 2], dx * b.z); a2 = fmaf(s[4 * i + 2], c.z, a2);
                    s[4 * i + 3] = fmaf(decay, s[4 * i + 3], dx * b.w); a3 = fmaf(s[4 * i + 3], c.w, a3);
                }
                float acc = (a0 + a1) + (a2 + a3);
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                acc += __shfl_xor_sync(0xffffffffu, acc, 4);
                if (live && j == 0) y[(size_t)(first + t0 + tt) * inner + h * P + p] = FIXED ? acc : fmaf(skip, x, acc);
            };
            // a whole chunk is unrolled so that a token's loads from shared memory are under way while the token before
            // it is still being summed over its lanes; the arithmetic and its order are the same either way
            constexpr int UNROLL = SCAN_UNROLL;
            if (cnt == CHUNK) {
#pragma unroll UNROLL
                for (int tt = 0; tt < CHUNK; ++tt) token(tt);
            } else {
                for (int tt = 0; tt < cnt; ++tt) token(tt);
            }
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) { const int n = ((i >> 2) * SCAN_LANES + j) * 4 + (i & 3); if (n < N) S[(size_t)n * P] = s[i]; }
    }
}

// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long ld_z,
                                           const float* __restrict__ w, T* __restrict__ out, int inner, int parts, float eps,
                                           int gate_after, int sigmoid_gate) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    const int t = blockIdx.x, part = blockIdx.y, width = inner / parts;
    const float* yr = y + (size_t)t * inner + (size_t)part * width;
    const T* zr = z + (size_t)t * ld_z + (size_t)part * width;
    float ss = 0.f;
    auto gate = [&](float z) { return sigmoid_gate ? 1.0f / (1.0f + expf(-z)) : silu_f(z); };
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = gate_after ? yr[i] : yr[i] * gate(pb_ld(zr + i)); ss += v * v; }
    ss = pb_warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nwarp; ++i) total += red[i];
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    T* o = out + (size_t)t * inner + (size_t)part * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        pb_st(o + i, yr[i] * gate(pb_ld(zr + i)) * inv * w[(size_t)part * width + i]);   // the same product either way
}

template <typename TI, typename TO>
__global__ void scaled_sum_kernel(const TI* __restrict__ a, float sa, const TI* __restrict__ b, float sb, TO* __restrict__ out, long long n) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pb_st(out + i, sa * pb_ld(a + i) + sb * pb_ld(b + i));
}

}  // namespace

// in: the step's [x | B | C] columns of the input projection, [n_tokens, channels] with row stride ld_in; w float32
// [channels, taps] (last column: the current token); carried [slots, taps - 1, channels]; out [n_tokens, channels] dense.
PB_API int pb_causal_conv_silu(const void* in, long long ld_in, const float* w, const float* bias, const void* carried, void* out,
                               int dtype, const int32_t* token_seq, const int32_t* positions, const int32_t* q_start,
                               const int32_t* slots, int n_tokens, int channels, int taps, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && channels > 0 && taps >= 1 && ld_in >= channels, "causal_conv_silu: bad sizes");
    PB_REQUIRE(in && w && out && token_seq && positions && q_start && slots && (taps == 1 || carried), "causal_conv_silu: null pointer");
    if (n_tokens == 0) return 0;
    PB_REQUIRE((channels + 127) / 128 < 65536, "causal_conv_silu: %d channels in one launch", channels);
    const int vn = dtype == PB_BF16 ? 8 : 4;
    if (taps >= 2 && taps <= 4 && channels % vn == 0 && ld_in % vn == 0 && pb_aligned(in, 16) && pb_aligned(out, 16) && pb_aligned(carried, 16)) {
        const int run = n_tokens <= 64 ? 1 : CONV_RUN;
        const dim3 grid((n_tokens + run - 1) / run, (channels / vn + 63) / 64);
#define CONV_LAUNCH(TAPS)                                                                                                     \
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(causal_conv_silu_vec_kernel<T, TAPS>, grid, dim3(64), 0, stream, (const T*)in, ld_in, w, bias, \
                                           (const T*)carried, (T*)out, token_seq, positions, q_start, slots, n_tokens, channels, run)))
        if (taps == 2) CONV_LAUNCH(2);
        else if (taps == 3) CONV_LAUNCH(3);
        else CONV_LAUNCH(4);
#undef CONV_LAUNCH
        PB_CHECK_LAUNCH("causal_conv_silu");
        return 0;
    }
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(causal_conv_silu_kernel<T>, dim3(n_tokens, (channels + 127) / 128), dim3(128), 0, stream, (const T*)in, ld_in, w, bias,
                   (const T*)carried, (T*)out, token_seq, positions, q_start, slots, n_tokens, channels, taps)));
    PB_CHECK_LAUNCH("causal_conv_silu");
    return 0;
}

// cu_q [n_seqs + 1], slots [n_seqs]: a sequence whose length cu_q[r + 1] - cu_q[r] is not positive is skipped.
PB_API int pb_conv_state_update(const void* in, long long ld_in, void* carried, int dtype, const int32_t* cu_q, const int32_t* slots,
                                int n_seqs, int channels, int taps, cudaStream_t stream) {
    PB_REQUIRE(n_seqs >= 0 && channels > 0 && taps >= 1 && ld_in >= channels, "conv_state_update: bad sizes");
    if (n_seqs == 0 || taps == 1) return 0;
    PB_REQUIRE(in && carried && cu_q && slots, "conv_state_update: null pointer");
    PB_REQUIRE(n_seqs < 65536, "conv_state_update: %d sequences in one launch", n_seqs);
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(conv_state_update_kernel<T>, dim3((channels + 127) / 128, n_seqs), dim3(128), 0, stream, (const T*)in, ld_in,
                   (T*)carried, cu_q, slots, channels, taps)));
    PB_CHECK_LAUNCH("conv_state_update");
    return 0;
}

// u: the convolution's output [n_tokens, heads * P + 2 * groups * N] dense, laid out [x | B | C]; dt_in: the step-size
// columns of the input projection, row stride ld_dt; state float32 [slots, heads, N, P]; y float32 [n_tokens, heads * P].
PB_API int pb_ssm_scan(const void* u, const void* dt_in, long long ld_dt, int dtype, const float* dt_bias, const float* a_log,
                       const float* d_skip, float* state, float* y, const int32_t* cu_q, const int32_t* slots, int n_seqs,
                       int heads, int P, int N, int groups, cudaStream_t stream) {
    PB_REQUIRE(n_seqs >= 0 && heads > 0 && P > 0 && N > 0 && groups > 0 && heads % groups == 0, "ssm_scan: bad sizes");
    PB_REQUIRE(N <= 32 * SCAN_LANES, "ssm_scan: a state of %d rows (at most %d)", N, 32 * SCAN_LANES);
    PB_REQUIRE(u && dt_in && dt_bias && a_log && d_skip && state && y && cu_q && slots && ld_dt >= heads, "ssm_scan: null pointer");
    if (n_seqs == 0) return 0;
    PB_REQUIRE(n_seqs < 65536, "ssm_scan: %d sequences in one launch", n_seqs);
    const int col_blocks = (P + SCAN_COLS - 1) / SCAN_COLS;
    const dim3 grid(heads * col_blocks, n_seqs), block(2 * SCAN_COLS * SCAN_LANES);
    const int npl = (N + SCAN_LANES - 1) / SCAN_LANES;
#define SCAN_LAUNCH(NPL)                                                                                                    \
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(ssm_scan_kernel<T, NPL, false>, grid, block, 0, stream, (const T*)u,               \
                                           (long long)(heads * P + 2 * groups * N), (const T*)dt_in, ld_dt, dt_bias, a_log, d_skip,  \
                                           state, y, cu_q, slots, heads, P, N, groups, 0)))
    if (npl <= 4) SCAN_LAUNCH(4);
    else if (npl <= 8) SCAN_LAUNCH(8);
    else if (npl <= 16) SCAN_LAUNCH(16);
    else SCAN_LAUNCH(32);
#undef SCAN_LAUNCH
    PB_CHECK_LAUNCH("ssm_scan");
    return 0;
}

// Linear attention with a decaying state: per head S <- decay_h S + k v^T, o = S^T q, with q, k, v the SiLU of the
// projection's columns.  u: the projection, rows ld_u apart, laid out [v: heads * P | k: heads * N | q: heads * N];
// decay float32 [heads]; state float32 [slots, heads, N, P]; y float32 [n_tokens, heads * P].  activated: the columns
// hold silu(v), silu(k), silu(q) already (pb_silu_cols), the scan takes them as they are.
PB_API int pb_decay_scan(const void* u, long long ld_u, int dtype, const float* decay, float* state, float* y, const int32_t* cu_q,
                         const int32_t* slots, int n_seqs, int heads, int P, int N, int activated, cudaStream_t stream) {
    PB_REQUIRE(n_seqs >= 0 && heads > 0 && P > 0 && N > 0 && ld_u >= (long long)heads * (P + 2 * N), "decay_scan: bad sizes");
    PB_REQUIRE(N <= 32 * SCAN_LANES, "decay_scan: keys of %d elements (at most %d)", N, 32 * SCAN_LANES);
    PB_REQUIRE(u && decay && state && y && cu_q && slots, "decay_scan: null pointer");
    if (n_seqs == 0) return 0;
    PB_REQUIRE(n_seqs < 65536, "decay_scan: %d sequences in one launch", n_seqs);
    const int col_blocks = (P + SCAN_COLS - 1) / SCAN_COLS;
    const dim3 grid(heads * col_blocks, n_seqs), block(2 * SCAN_COLS * SCAN_LANES);
    const int npl = (N + SCAN_LANES - 1) / SCAN_LANES;
#define SCAN_LAUNCH(NPL)                                                                                                    \
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(ssm_scan_kernel<T, NPL, true>, grid, block, 0, stream, (const T*)u, ld_u, (const T*)nullptr, \
                                           0ll, (const float*)nullptr, decay, (const float*)nullptr, state, y, cu_q, slots, heads, P, \
                                           N, heads, activated ? 0 : 1)))
    if (npl <= 4) SCAN_LAUNCH(4);
    else if (npl <= 8) SCAN_LAUNCH(8);
    else if (npl <= 16) SCAN_LAUNCH(16);
    else SCAN_LAUNCH(32);
#undef SCAN_LAUNCH
    PB_CHECK_LAUNCH("decay_scan");
    return 0;
}

// y float32 [n_tokens, inner]; z: the gate columns of the input projection, row stride ld_z; w float32 [inner];
// out [n_tokens, inner] dense.  gate_after 0: norm(y * gate(z)) * w; 1: norm(y) * w * gate(z); gate is SiLU, or the
// sigmoid with sigmoid_gate.
PB_API int pb_gated_group_rmsnorm(const float* y, const void* z, long long ld_z, const float* w, void* out, int dtype, int n_tokens,
                                  int inner, int parts, float eps, int gate_after, int sigmoid_gate, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && inner > 0 && parts > 0 && inner % parts == 0 && ld_z >= inner, "gated_group_rmsnorm: bad sizes");
    PB_REQUIRE(y && z && w && out, "gated_group_rmsnorm: null pointer");
    if (n_tokens == 0) return 0;
    PB_REQUIRE(parts < 65536, "gated_group_rmsnorm: %d parts", parts);
    int threads = 32;
    while (threads < 256 && threads < inner / parts) threads <<= 1;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(gated_group_rmsnorm_kernel<T>, dim3(n_tokens, parts), dim3(threads), 0, stream, y, (const T*)z, ld_z, w, (T*)out, inner,
                   parts, eps, gate_after, sigmoid_gate)));
    PB_CHECK_LAUNCH("gated_group_rmsnorm");
    return 0;
}

// out = sa * a + sb * b, element by element in float32; a and b of type in_dtype, out of out_dtype.
PB_API int pb_scaled_sum(const void* a, float sa, const void* b, float sb, void* out, int in_dtype, int out_dtype, long long n,
                         cudaStream_t stream) {
    PB_REQUIRE(n >= 0 && a && b && out, "scaled_sum: bad arguments");
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == PB_F32 && out_dtype == PB_F32)
        pb_launch(scaled_sum_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)a, sa, (const float*)b, sb, (float*)out, n);
    else if (in_dtype == PB_F32 && out_dtype == PB_BF16)
        pb_launch(scaled_sum_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const float*)a, sa, (const float*)b, sb,
                  (__nv_bfloat16*)out, n);
    else if (in_dtype == PB_BF16 && out_dtype == PB_BF16)
        pb_launch(scaled_sum_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)a, sa,
                  (const __nv_bfloat16*)b, sb, (__nv_bfloat16*)out, n);
    else
        return pb_fail("scaled_sum: unsupported types in=%d out=%d", in_dtype, out_dtype);
    PB_CHECK_LAUNCH("scaled_sum");
    return 0;
}
