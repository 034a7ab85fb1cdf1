// Paged softmax attention on the tensor cores (bfloat16 operands, float32 sums) for the shapes the plain attention
// kernels do not take: keys and values of different sizes, values that are the first `vd` elements of the cached key
// rows (a latent that is key and value at once, hundreds of elements long, shared by all query heads), a window, first
// tokens that stay visible behind the window, chunks, capped scores, a sink per head, a gate per (token, head).  Prompt
// portions and decoded tokens alike.
//
// A block works on 32 query rows - the heads of one key/value head's group for as many consecutive tokens of one
// request as fit (32 / heads), or 32 of one token's heads - against tiles of 32 keys aligned to absolute positions.
// Eight warps: warp (r, c) owns rows 16 r .. 16 r + 15; it scores them against keys 8 c .. 8 c + 7 of the tile
// (S = Q K^T, mma.sync m16n8k16, Q and K from shared memory by ldmatrix), the four warps of a row exchange their
// maxima and sums through shared memory, the weights go to shared memory as bfloat16, and the warp adds
// P V for its quarter of the value columns (so a 512-wide value costs a thread 64 accumulators, not 256).  K tiles
// arrive by 16-byte cp.async; two blocks share a multiprocessor, one loading while the other multiplies.  With
// `splits` > 1 the key tiles of a block's rows are dealt to that many blocks, which leave (maximum, sum, unnormalised
// output) in scratch memory for pb_attention_paged_tc_merge: a decode step's few rows fill the device that way.
// The sink joins the denominator where the parts are put together (here, or in the merge).
//
// Takes kd % 16 == 0, vd % 32 == 0, vd <= 512, as many value heads as key heads, pages without permuted chunks.
#include "common.cuh"

#include <math.h>

namespace {

typedef __nv_bfloat16 bf16;

#define TC_ROWS 32
#define TC_KEYS 32
#define TC_PLD 40            // row stride of the weights in shared memory (elements)

struct TcParams {
    const bf16* q;
    const bf16* k_pages;
    const bf16* v_pages;
    bf16* out;
    const float* sink;
    const int32_t* positions;
    const int32_t* table_row;
    const int32_t* block_table;
    const int32_t* cu_q;
    const int32_t* tile_seq;
    const int32_t* tile_tok0;
    float* part_o;
    float* part_ml;
    int table_stride, page_size, num_pages, n_tokens, H, G, kd, vd, v_row, v_shared, window, splits, hp, tpt, head_tiles;
    int keep_first, chunk;        // positions below keep_first stay visible behind a window; chunk > 0: keys of the query's own run only
    float scale, softcap;         // softcap > 0: score = softcap * tanh(score / softcap)
    const bf16* gate;             // [n_tokens, H] with row stride ld_gate, or null: sigmoid(gate) multiplies the head's output
    long long ld_gate;
    int* status;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned (&r)[2], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int NT_MAX>
__global__ void __launch_bounds__(256, 2) attention_paged_tc_kernel(TcParams p) {
    pb_grid_dep_launch();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = warp & 1, c = warp >> 1;
    const int kd = p.kd, vd = p.vd, ldk = kd + 8, ldv = p.v_shared ? ldk : vd + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + TC_ROWS * ldk;
    bf16* Vs = p.v_shared ? Ks : Ks + TC_KEYS * ldk;
    bf16* Ps = p.v_shared ? Ks + TC_KEYS * ldk : Vs + TC_KEYS * ldv;
    float* m_part = reinterpret_cast<float*>(Ps + TC_ROWS * TC_PLD);      // [32][4]
    float* l_part = m_part + TC_ROWS * 4;
    int* row_pos = reinterpret_cast<int*>(l_part + TC_ROWS * 4);          // the row's position, -1: no such row
    int* row_q = row_pos + TC_ROWS;                                       // token * H + head
    int* key_page = row_q + TC_ROWS;

    const int group = p.H / p.G;
    const int g = blockIdx.y / p.head_tiles, ht = blockIdx.y % p.head_tiles;
    const int z = blockIdx.z;
    pb_grid_dep_wait();
    int tok_first, n_tok;
    if (p.tile_seq != nullptr) {
        const int s = p.tile_seq[blockIdx.x], t0 = p.tile_tok0[blockIdx.x];
        tok_first = p.cu_q[s] + t0;
        n_tok = min(p.tpt, p.cu_q[s + 1] - p.cu_q[s] - t0);
    } else {
        tok_first = blockIdx.x;
        n_tok = 1;
    }
    const int trow = p.table_row[tok_first];
    if (trow < 0 || n_tok <= 0) return;                                   // a padding row of a captured step
    const int32_t* table = p.block_table + (size_t)trow * p.table_stride;
    const int p0 = p.positions[tok_first], p1 = p.positions[tok_first + n_tok - 1];
    const int lo_tile = p.window > 0 ? max(0, p0 - p.window + 1) : (p.chunk > 0 ? p0 - p0 % p.chunk : 0);
    const int first_kt = lo_tile / TC_KEYS, last_kt = p1 / TC_KEYS;
    // the tiles of the kept first tokens that lie wholly before the first tile of the rows' own range come first; the
    // walk below counts both runs through (index v -> tile kt_of(v))
    const int keep_tiles = p.window > 0 ? min((min(p.keep_first, lo_tile) + TC_KEYS - 1) / TC_KEYS, first_kt) : 0;
    const int n_walk = keep_tiles + last_kt - first_kt + 1;
    const int per_split = (n_walk + p.splits - 1) / p.splits;
    const int kt_begin = z * per_split, kt_end = min(n_walk, kt_begin + per_split);
    auto kt_of = [&](int v) { return v < keep_tiles ? v : first_kt + (v - keep_tiles); };
    auto in_range = [&](int j) { return j <= p1 && (j >= lo_tile || j < p.keep_first); };

    if (tid < TC_ROWS) {
        const int ti = tid / p.hp, hi = tid % p.hp;
        const bool valid = tid < p.tpt * p.hp && ti < n_tok && ht * p.hp + hi < group;
        const int t = tok_first + ti;
        row_pos[tid] = valid ? p.positions[t] : -1;
        row_q[tid] = valid ? t * p.H + g * group + ht * p.hp + hi : -1;
        const int j = kt_of(kt_begin) * TC_KEYS + tid;
        int page = (kt_begin < kt_end && in_range(j)) ? table[j / p.page_size] : -1;
        if (page >= p.num_pages) { page = -1; if (p.status) atomicExch(p.status, 6); }
        key_page[tid] = page;
    }
    __syncthreads();
    const int kchunks = kd >> 3, vchunks = vd >> 3;
    const int ld_row = tid >> 3, ld_sub = tid & 7;                         // eight threads copy a row, 16 bytes at a time
    {
        bf16* dst = Qs + ld_row * ldk;
        if (row_q[ld_row] >= 0) {
            const bf16* src = p.q + (size_t)row_q[ld_row] * kd;
            for (int ch = ld_sub; ch < kchunks; ch += 8) cp_async16(dst + ch * 8, src + ch * 8);
        } else {
            for (int ch = ld_sub; ch < kchunks; ch += 8) *reinterpret_cast<uint4*>(dst + ch * 8) = make_uint4(0, 0, 0, 0);
        }
    }

    const int row0 = r * 16 + (lane >> 2), row1 = row0 + 8;
    const int keyc = c * 8 + (lane & 3) * 2;
    const int nt_n = vd >> 5;                                             // n8 tiles of this warp's quarter of the columns
    const int col0 = c * (vd >> 2);
    float o[NT_MAX][4];
#pragma unroll
    for (int i = 0; i < NT_MAX; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int kbase = kt_of(kt) * TC_KEYS;
        {
            const int page = key_page[ld_row];
            const int in_page = (kbase + ld_row) % p.page_size;
            bf16* dst = Ks + ld_row * ldk;
            if (page >= 0) {
                const bf16* src = p.k_pages + (((size_t)page * p.G + g) * p.page_size + in_page) * kd;
                for (int ch = ld_sub; ch < kchunks; ch += 8) cp_async16(dst + ch * 8, src + ch * 8);
            } else {
                for (int ch = ld_sub; ch < kchunks; ch += 8) *reinterpret_cast<uint4*>(dst + ch * 8) = make_uint4(0, 0, 0, 0);
            }
            if (!p.v_shared) {
                bf16* vdst = Vs + ld_row * ldv;
                if (page >= 0) {
                    const bf16* src = p.v_pages + (((size_t)page * p.G + g) * p.page_size + in_page) * p.v_row;
                    for (int ch = ld_sub; ch < vchunks; ch += 8) cp_async16(vdst + ch * 8, src + ch * 8);
                } else {
                    for (int ch = ld_sub; ch < vchunks; ch += 8) *reinterpret_cast<uint4*>(vdst + ch * 8) = make_uint4(0, 0, 0, 0);
                }
            }
        }
        cp_async_wait_all();
        __syncthreads();                                                   // (1) the tile (and, the first time, Q) is there

        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            // four chains of products, one after the other in k: a single accumulator would make every product wait for
            // the one before it
            float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f}, s3[4] = {0.f, 0.f, 0.f, 0.f};
            const bf16* a_ptr = Qs + (r * 16 + (lane & 15)) * ldk + (lane >> 4) * 8;
            const bf16* b_ptr = Ks + (c * 8 + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8;
            int kk = 0;
            for (; kk + 64 <= kd; kk += 64) {
                unsigned a0[4], a1[4], a2[4], a3[4], b0[2], b1[2], b2[2], b3[2];
                ldmatrix_x4(a0, a_ptr + kk);
                ldmatrix_x2(b0, b_ptr + kk);
                ldmatrix_x4(a1, a_ptr + kk + 16);
                ldmatrix_x2(b1, b_ptr + kk + 16);
                ldmatrix_x4(a2, a_ptr + kk + 32);
                ldmatrix_x2(b2, b_ptr + kk + 32);
                ldmatrix_x4(a3, a_ptr + kk + 48);
                ldmatrix_x2(b3, b_ptr + kk + 48);
                mma_bf16(s, a0, b0);
                mma_bf16(s1, a1, b1);
                mma_bf16(s2, a2, b2);
                mma_bf16(s3, a3, b3);
            }
            for (; kk < kd; kk += 16) {
                unsigned a[4], b[2];
                ldmatrix_x4(a, a_ptr + kk);
                ldmatrix_x2(b, b_ptr + kk);
                mma_bf16(s, a, b);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] = (s[e] + s1[e]) + (s2[e] + s3[e]);
        }
        const int pos0 = row_pos[row0], pos1 = row_pos[row1];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int pos = e < 2 ? pos0 : pos1;
            const int key = keyc + (e & 1), j = kbase + key;
            const bool ok = pos >= 0 && j <= pos && (p.window <= 0 || j > pos - p.window || j < p.keep_first) &&
                            (p.chunk <= 0 || j >= pos - pos % p.chunk) && key_page[key] >= 0;
            const float sc = s[e] * p.scale;
            s[e] = ok ? (p.softcap > 0.f ? p.softcap * tanhf(sc / p.softcap) : sc) : -INFINITY;
        }
        const float mx0 = quad_max(fmaxf(s[0], s[1])), mx1 = quad_max(fmaxf(s[2], s[3]));
        if ((lane & 3) == 0) { m_part[row0 * 4 + c] = mx0; m_part[row1 * 4 + c] = mx1; }
        __syncthreads();                                                   // (2) the four warps of a row know each other's maxima
        const float mt0 = fmaxf(fmaxf(m_part[row0 * 4], m_part[row0 * 4 + 1]), fmaxf(m_part[row0 * 4 + 2], m_part[row0 * 4 + 3]));
        const float mt1 = fmaxf(fmaxf(m_part[row1 * 4], m_part[row1 * 4 + 1]), fmaxf(m_part[row1 * 4 + 2], m_part[row1 * 4 + 3]));
        const float mn0 = fmaxf(m0, mt0), mn1 = fmaxf(m1, mt1);
        const float u0 = mn0 == -INFINITY ? 0.f : mn0, u1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = m0 == -INFINITY ? 0.f : expf(m0 - u0), corr1 = m1 == -INFINITY ? 0.f : expf(m1 - u1);
        const float e0 = expf(s[0] - u0), e1 = expf(s[1] - u0), e2 = expf(s[2] - u1), e3 = expf(s[3] - u1);
        const float ls0 = quad_sum(e0 + e1), ls1 = quad_sum(e2 + e3);
        if ((lane & 3) == 0) { l_part[row0 * 4 + c] = ls0; l_part[row1 * 4 + c] = ls1; }
        *reinterpret_cast<__nv_bfloat162*>(Ps + row0 * TC_PLD + keyc) = __floats2bfloat162_rn(e0, e1);
        *reinterpret_cast<__nv_bfloat162*>(Ps + row1 * TC_PLD + keyc) = __floats2bfloat162_rn(e2, e3);
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int i = 0; i < NT_MAX; ++i) {
            if (i < nt_n) { o[i][0] *= corr0; o[i][1] *= corr0; o[i][2] *= corr1; o[i][3] *= corr1; }
        }
        __syncthreads();                                                   // (3) weights and sums of the tile are there
        l0 = l0 * corr0 + ((l_part[row0 * 4] + l_part[row0 * 4 + 1]) + (l_part[row0 * 4 + 2] + l_part[row0 * 4 + 3]));
        l1 = l1 * corr1 + ((l_part[row1 * 4] + l_part[row1 * 4 + 1]) + (l_part[row1 * 4 + 2] + l_part[row1 * 4 + 3]));
#pragma unroll
        for (int ks = 0; ks < TC_KEYS / 16; ++ks) {
            unsigned a[4];
            ldmatrix_x4(a, Ps + (r * 16 + (lane & 15)) * TC_PLD + ks * 16 + (lane >> 4) * 8);
            const bf16* v_ptr = Vs + (ks * 16 + (lane & 15)) * ldv + col0;
#pragma unroll
            for (int i = 0; i < NT_MAX; ++i) {
                if (i < nt_n) {
                    unsigned b[2];
                    ldmatrix_x2_trans(b, v_ptr + i * 8);
                    mma_bf16(o[i], a, b);
                }
            }
        }
        if (tid < TC_KEYS) {                                              // the next tile's pages
            const int j = kt_of(kt + 1) * TC_KEYS + tid;
            int page = (kt + 1 < kt_end && in_range(j)) ? table[j / p.page_size] : -1;
            if (page >= p.num_pages) { page = -1; if (p.status) atomicExch(p.status, 6); }
            // written after everybody has read this tile's entries: they were last read before barrier (3)
            key_page[tid] = page;
        }
        __syncthreads();                                                   // (4) everybody is done with the tile
    }
    if (kt_begin >= kt_end) { cp_async_wait_all(); }

    const int q0 = row_q[row0], q1 = row_q[row1];
    if (p.splits > 1) {
        if (q0 >= 0) {
            float* dst = p.part_o + ((size_t)q0 * p.splits + z) * vd + col0 + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < NT_MAX; ++i) if (i < nt_n) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][0], o[i][1]);
            if (c == 0 && (lane & 3) == 0) { float* ml = p.part_ml + ((size_t)q0 * p.splits + z) * 2; ml[0] = m0; ml[1] = l0; }
        }
        if (q1 >= 0) {
            float* dst = p.part_o + ((size_t)q1 * p.splits + z) * vd + col0 + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < NT_MAX; ++i) if (i < nt_n) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2], o[i][3]);
            if (c == 0 && (lane & 3) == 0) { float* ml = p.part_ml + ((size_t)q1 * p.splits + z) * 2; ml[0] = m1; ml[1] = l1; }
        }
        return;
    }
    float f0 = 1.f, f1 = 1.f;
    if (p.sink != nullptr) {                                              // one more term of the denominator, no key, no value
        if (q0 >= 0) { const float sk = p.sink[q0 % p.H], mf = fmaxf(m0, sk); f0 = m0 == -INFINITY ? 0.f : expf(m0 - mf); l0 = l0 * f0 + expf(sk - mf); }
        if (q1 >= 0) { const float sk = p.sink[q1 % p.H], mf = fmaxf(m1, sk); f1 = m1 == -INFINITY ? 0.f : expf(m1 - mf); l1 = l1 * f1 + expf(sk - mf); }
    }
    float inv0 = l0 > 0.f ? f0 / l0 : 0.f, inv1 = l1 > 0.f ? f1 / l1 : 0.f;
    if (p.gate != nullptr) {
        if (q0 >= 0) inv0 *= 1.0f / (1.0f + expf(-__bfloat162float(p.gate[(size_t)(q0 / p.H) * p.ld_gate + q0 % p.H])));
        if (q1 >= 0) inv1 *= 1.0f / (1.0f + expf(-__bfloat162float(p.gate[(size_t)(q1 / p.H) * p.ld_gate + q1 % p.H])));
    }
    if (q0 >= 0) {
        bf16* dst = p.out + (size_t)q0 * vd + col0 + (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < NT_MAX; ++i) if (i < nt_n) *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][0] * inv0, o[i][1] * inv0);
    }
    if (q1 >= 0) {
        bf16* dst = p.out + (size_t)q1 * vd + col0 + (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < NT_MAX; ++i) if (i < nt_n) *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2] * inv1, o[i][3] * inv1);
    }
}

// One block per (token, head): the parts of its key ranges, the sink, the division.  The parts' weights
// exp(m_s - M) / L are made once, by the first warp; then every thread adds up its columns, the loads of all parts
// in flight together.
#define TC_MAX_SPLITS 64
__global__ void __launch_bounds__(128) attention_paged_tc_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                       const float* __restrict__ sink, const int32_t* __restrict__ table_row,
                                                                       const bf16* __restrict__ gate, long long ld_gate,
                                                                       bf16* __restrict__ out, int H, int vd, int splits) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float w_s[TC_MAX_SPLITS];
    const int row = blockIdx.x;
    if (table_row[row / H] < 0) return;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float* ml = part_ml + (size_t)row * splits * 2;
        const float ma = lane < splits ? ml[2 * lane] : -INFINITY, mb = lane + 32 < splits ? ml[2 * (lane + 32)] : -INFINITY;
        const float la = lane < splits ? ml[2 * lane + 1] : 0.f, lb = lane + 32 < splits ? ml[2 * (lane + 32) + 1] : 0.f;
        const float sk = sink ? sink[row % H] : -INFINITY;
        const float M = fmaxf(pb_warp_max(fmaxf(ma, mb)), sk);
        const float wa = ma == -INFINITY ? 0.f : expf(ma - M), wb = mb == -INFINITY ? 0.f : expf(mb - M);
        const float L = pb_warp_sum(la * wa + lb * wb) + (sink ? expf(sk - M) : 0.f);
        float inv = L > 0.f ? 1.0f / L : 0.f;
        if (gate != nullptr) inv *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)(row / H) * ld_gate + row % H])));
        w_s[lane] = wa * inv;
        w_s[lane + 32] = wb * inv;
    }
    __syncthreads();
    const float* po = part_o + (size_t)row * splits * vd;
    for (int d = threadIdx.x * 4; d < vd; d += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(po + (size_t)s * vd + d);
            const float w = w_s[s];
            acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y); acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
        }
        bf16* o = out + (size_t)row * vd + d;
        *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(acc.x, acc.y);
        *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(acc.z, acc.w);
    }
}

size_t tc_smem(int kd, int vd, int v_shared) {
    const size_t ldk = kd + 8, ldv = vd + 8;
    return (TC_ROWS * ldk + TC_KEYS * ldk + (v_shared ? 0 : TC_KEYS * ldv) + TC_ROWS * TC_PLD) * sizeof(bf16) + TC_ROWS * 4 * 2 * sizeof(float) +
           3 * TC_ROWS * sizeof(int);
}

}  // namespace

PB_API int pb_attention_paged_tc_supported(int H, int G, int kd, int vd, int v_shared) {
    if (H <= 0 || G <= 0 || H % G) return 0;
    if (kd % 16 || vd % 32 || vd > 512 || kd <= 0 || vd <= 0) return 0;
    if (v_shared && vd > kd) return 0;
    return tc_smem(kd, vd, v_shared) <= 110 * 1024 ? 1 : 0;
}

// Tokens of one request that a block takes at a time: what the caller's list of tiles is made with.
PB_API int pb_attention_paged_tc_tile_tokens(int H, int G) {
    const int group = H / G;
    return group >= TC_ROWS ? 1 : TC_ROWS / group;
}

PB_API long long pb_attention_paged_tc_scratch_floats(int n_tokens, int H, int vd, int splits) {
    return splits > 1 ? (long long)n_tokens * H * splits * (vd + 2) : 0;
}

// q [n_tokens, H, kd], out [n_tokens, H, vd], pages [num_pages, G, page_size, kd] (values: [.., v_row], or the key pages
// themselves with v_shared); tiles: tile_seq/tile_tok0 [n_tiles] (request of the batch, first token within its portion) with
// cu_q, or null: tile i is token i alone (a step of single tokens).  scratch: float32 of pb_attention_paged_tc_scratch_floats.
// window, keep_first, chunk, softcap, gate: as for pb_attention_paged.
PB_API int pb_attention_paged_tc_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const float* sink,
                                      const int32_t* positions, const int32_t* table_row, const int32_t* block_table, int table_stride,
                                      const int32_t* cu_q, const int32_t* tile_seq, const int32_t* tile_tok0, int n_tiles, int page_size,
                                      int num_pages, int n_tokens, int H, int G, int kd, int vd, int v_row, int v_shared, float scale,
                                      int window, int keep_first, int chunk, float softcap, const void* gate, long long ld_gate,
                                      int splits, float* scratch, int* status, cudaStream_t stream) {
    PB_REQUIRE(pb_attention_paged_tc_supported(H, G, kd, vd, v_shared), "attention_paged_tc: shape H=%d G=%d kd=%d vd=%d not taken", H, G, kd, vd);
    PB_REQUIRE(q && k_pages && v_pages && out && positions && table_row && block_table, "attention_paged_tc: null pointer");
    PB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0 && n_tiles >= 0 && n_tokens >= 0, "attention_paged_tc: bad geometry");
    PB_REQUIRE(tile_seq == nullptr || (tile_tok0 && cu_q), "attention_paged_tc: a list of tiles needs the portions' offsets");
    PB_REQUIRE(keep_first >= 0 && chunk >= 0 && !(window > 0 && chunk > 0) && (gate == nullptr || ld_gate >= H),
               "attention_paged_tc: window %d, kept %d, chunk %d", window, keep_first, chunk);
    PB_REQUIRE(splits >= 1 && splits <= TC_MAX_SPLITS && (splits == 1 || (scratch && pb_aligned(scratch, 16))), "attention_paged_tc: %d splits", splits);
    PB_REQUIRE(pb_aligned(q, 16) && pb_aligned(k_pages, 16) && pb_aligned(v_pages, 16) && pb_aligned(out, 4) && (v_shared || v_row % 8 == 0),
               "attention_paged_tc: operands must be 16-byte aligned");
    if (n_tiles == 0) return 0;
    const int group = H / G;
    TcParams p;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages; p.out = (bf16*)out; p.sink = sink;
    p.positions = positions; p.table_row = table_row; p.block_table = block_table; p.cu_q = cu_q; p.tile_seq = tile_seq; p.tile_tok0 = tile_tok0;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * H * splits * vd : nullptr;
    p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages; p.n_tokens = n_tokens; p.H = H; p.G = G; p.kd = kd; p.vd = vd;
    p.v_row = v_shared ? kd : v_row; p.v_shared = v_shared; p.window = window; p.splits = splits;
    p.hp = group >= TC_ROWS ? TC_ROWS : group;
    p.tpt = tile_seq ? TC_ROWS / p.hp : 1;
    p.head_tiles = (group + p.hp - 1) / p.hp;
    p.scale = scale; p.status = status;
    p.keep_first = window > 0 ? keep_first : 0; p.chunk = chunk; p.softcap = softcap; p.gate = (const bf16*)gate; p.ld_gate = ld_gate;
    const size_t smem = tc_smem(kd, vd, v_shared);
    const dim3 grid(n_tiles, G * p.head_tiles, splits);
    PB_REQUIRE(G * p.head_tiles < 65536, "attention_paged_tc: too many head tiles");
    const int nt = vd / 32;
#define TC_LAUNCH(NT)                                                                                                        \
    do {                                                                                                                     \
        static bool set = false;                                                                                             \
        if (!set) {                                                                                                          \
            cudaFuncSetAttribute(attention_paged_tc_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);    \
            set = true;                                                                                                      \
        }                                                                                                                    \
        pb_launch(attention_paged_tc_kernel<NT>, grid, dim3(256), smem, stream, p);                                          \
    } while (0)
    if (nt <= 2) TC_LAUNCH(2);
    else if (nt <= 4) TC_LAUNCH(4);
    else if (nt <= 8) TC_LAUNCH(8);
    else TC_LAUNCH(16);
#undef TC_LAUNCH
    PB_CHECK_LAUNCH("attention_paged_tc");
    if (splits > 1) {
        pb_launch(attention_paged_tc_merge_kernel, dim3(n_tokens * H), dim3(128), 0, stream, (const float*)p.part_o, (const float*)p.part_ml, sink,
                  table_row, (const bf16*)gate, ld_gate, (bf16*)out, H, vd, splits);
        PB_CHECK_LAUNCH("attention_paged_tc_merge");
    }
    return 0;
}
