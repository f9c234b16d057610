// Attention over a cache of latents: every head reads the same vector c_j of R numbers per cached token, as its
// key and as its value.  The head's own key and value matrices are applied outside (to the query before, to the
// result after), so a token costs R cached numbers whatever the number of heads:
//
//     s_hj = scale * (q'_h . c_j),   p_h = softmax_j(s_hj) over the visible j,   ctx_h = sum_j p_hj c_j
//
// with q'_h = K_h^T q_h (the query taken through the head's key matrix) and the head's output V_h ctx_h.
// A token at position pos of its request sees j in lo..pos, lo = 0 or pos - window + 1.
//
// One block per (row, group of heads, slice of the keys): 32 latents at a time go to shared memory once for all
// heads of the group; a warp owns up to two heads; lane j scores key j, then every lane gathers its share of the R
// numbers of ctx.  Scores, the softmax and the sums are float in both builds.  Keys come in ascending order from a
// multiple of 32, so the order of every sum depends only on (pos, window, slices), never on the batch or the pages.
//
// With more than one slice of keys per row (long contexts in steps of few rows), every slice leaves its unscaled
// sum, maximum and denominator in a workspace and a second kernel joins them.
#include "common.cuh"

#define LA_WARPS 8
#define LA_HPW 2                       // heads per warp
#define LA_HEADS (LA_WARPS * LA_HPW)   // heads per block
#define LA_KEYS 32

template <typename QT, int RPL>  // latent numbers per lane: R <= 32 * RPL
__global__ void __launch_bounds__(32 * LA_WARPS)
latent_attention_kernel(const QT* __restrict__ q, long q_row, long q_head, const act_t* __restrict__ plane,
                        const int* __restrict__ block_table, int max_pages, int page_size, int n_pages,
                        const int* __restrict__ row_request, const int* __restrict__ positions, int n_heads, int R,
                        float scale, int window, int n_slices, act_t* __restrict__ out, long o_row, long o_head,
                        float* __restrict__ ws_acc, float* __restrict__ ws_ml) {
    extern __shared__ float smem[];
    const int ldt = R + 1;                       // a lane per key reads down a column: odd stride, no conflicts
    float* tile = smem;                          // [LA_KEYS][R + 1]
    float* qs = smem + LA_KEYS * ldt;            // [LA_HEADS][R]
    ib_grid_dependency_sync();
    const int row = blockIdx.x, slice = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head0 = blockIdx.y * LA_HEADS;
    const int pos = positions[row];
    const int req = row_request[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* bt = block_table + (long)req * max_pages;
    const int first = (lo / LA_KEYS) * LA_KEYS;
    const int n_tiles = (pos - first) / LA_KEYS + 1;
    const int per_slice = (n_tiles + n_slices - 1) / n_slices;
    const int t0 = slice * per_slice;
    const int t1 = min(n_tiles, t0 + per_slice);

    for (int i = threadIdx.x; i < LA_HEADS * R; i += blockDim.x) {
        const int h = head0 + i / R;
        qs[i] = h < n_heads ? ib_to_float(q[(long)row * q_row + (long)h * q_head + (i % R)]) * scale : 0.0f;
    }

    float acc[LA_HPW][RPL], m[LA_HPW], l[LA_HPW];
#pragma unroll
    for (int a = 0; a < LA_HPW; ++a) {
        m[a] = -INFINITY;
        l[a] = 0.0f;
#pragma unroll
        for (int k = 0; k < RPL; ++k) acc[a][k] = 0.0f;
    }

    for (int t = t0; t < t1; ++t) {
        const int j0 = first + t * LA_KEYS;
        __syncthreads();                         // the tile before has been used (and qs is written)
        for (int jj = warp; jj < LA_KEYS; jj += LA_WARPS) {
            const int j = j0 + jj;
            const act_t* src = nullptr;
            if (j >= lo && j <= pos) {
                const int page = bt[j / page_size];
                if (page >= 0 && page < n_pages) src = plane + ((long)page * page_size + (j % page_size)) * R;
            }
            for (int e = lane; e < R; e += 32) tile[jj * ldt + e] = src ? ib_to_float(src[e]) : 0.0f;
        }
        __syncthreads();
        const int j = j0 + lane;
        const bool valid = j >= lo && j <= pos;
        const int n_in_tile = min(LA_KEYS, pos - j0 + 1);
#pragma unroll
        for (int a = 0; a < LA_HPW; ++a) {
            const int hl = warp * LA_HPW + a;
            if (head0 + hl >= n_heads) continue;     // uniform over the warp
            const float* qh = qs + hl * R;
            float s = -INFINITY;
            if (valid) {
                const float* cj = tile + lane * ldt;
                float dot = 0.0f;
                for (int e = 0; e < R; ++e) dot = fmaf(qh[e], cj[e], dot);
                s = dot;
            }
            const float m_new = fmaxf(m[a], ib_warp_max(s));
            const float p = (s == -INFINITY) ? 0.0f : expf(s - m_new);
            const float corr = (m[a] == -INFINITY) ? 0.0f : expf(m[a] - m_new);
            l[a] = l[a] * corr + ib_warp_sum(p);
#pragma unroll
            for (int k = 0; k < RPL; ++k) acc[a][k] *= corr;
            for (int jj = 0; jj < n_in_tile; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                if (pj == 0.0f) continue;            // a key outside the window (uniform over the warp)
                const float* cv = tile + jj * ldt;
#pragma unroll
                for (int k = 0; k < RPL; ++k) {
                    const int e = lane + 32 * k;
                    if (e < R) acc[a][k] = fmaf(pj, cv[e], acc[a][k]);
                }
            }
            m[a] = m_new;
        }
    }
#pragma unroll
    for (int a = 0; a < LA_HPW; ++a) {
        const int h = head0 + warp * LA_HPW + a;
        if (h >= n_heads) continue;
        if (n_slices == 1) {
            const float inv = l[a] > 0.0f ? 1.0f / l[a] : 0.0f;
            act_t* dst = out + (long)row * o_row + (long)h * o_head;
#pragma unroll
            for (int k = 0; k < RPL; ++k) {
                const int e = lane + 32 * k;
                if (e < R) dst[e] = ib_from_float<act_t>(acc[a][k] * inv);
            }
        } else {
            const long item = ((long)row * n_heads + h) * n_slices + slice;
#pragma unroll
            for (int k = 0; k < RPL; ++k) {
                const int e = lane + 32 * k;
                if (e < R) ws_acc[item * R + e] = acc[a][k];
            }
            if (lane == 0) {
                ws_ml[item * 2] = m[a];
                ws_ml[item * 2 + 1] = l[a];
            }
        }
    }
}

// Joins the slices of one (row, head): a warp each.  A lane owns up to two slices' weights exp(m_s - m) (at most 64
// slices); the sums then run over the slices in ascending order with loads that carry no condition (a slice without
// keys has left zeros and the weight 0), so they are all under way together.
__global__ void latent_attention_join_kernel(const float* __restrict__ ws_acc, const float* __restrict__ ws_ml,
                                             int n_rows, int n_heads, int R, int n_slices, act_t* __restrict__ out,
                                             long o_row, long o_head) {
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)n_rows * n_heads) return;
    const int row = (int)(item / n_heads), h = (int)(item % n_heads);
    const float* ml = ws_ml + item * n_slices * 2;
    float ms[2], ls[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int s = min(lane + 32 * k, n_slices - 1);
        ms[k] = ml[s * 2];
        ls[k] = ml[s * 2 + 1];
        if (lane + 32 * k >= n_slices) { ms[k] = -INFINITY; ls[k] = 0.0f; }
    }
    const float m = ib_warp_max(fmaxf(ms[0], ms[1]));
    float w[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) w[k] = (ms[k] == -INFINITY) ? 0.0f : expf(ms[k] - m);
    const float l = ib_warp_sum(ls[0] * w[0] + ls[1] * w[1]);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    const float* acc = ws_acc + item * n_slices * R;
    act_t* dst = out + (long)row * o_row + (long)h * o_head;
    // all of a slice's numbers for this lane are asked for together (up to 16 loads under way), slice after slice
    float v[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = 0.0f;
#pragma unroll 2
    for (int s = 0; s < n_slices; ++s) {
        const float ws = __shfl_sync(0xffffffffu, s < 32 ? w[0] : w[1], s & 31);
        const float* a = acc + (long)s * R;
#pragma unroll
        for (int k = 0; k < 16; ++k) v[k] = fmaf(a[min(lane + 32 * k, R - 1)], ws, v[k]);
    }
#pragma unroll
    for (int k = 0; k < 16; ++k)
        if (lane + 32 * k < R) dst[lane + 32 * k] = ib_from_float<act_t>(v[k] * inv);
}

#if IB_ACT_BF16
// ---------------------------------------------------------------------------------------------------------------
// The same on the tensor cores (bfloat16 build; latents of a multiple of 32 numbers).  A block owns one row's group
// of up to 16 heads: the 16 x R queries are the A operand of both products.  Keys come 64 at a time by cp.async into
// one buffer (the shared memory then leaves room for two blocks per SM, which cover each other's waits).  Scores: every one of the four warps takes
// 16 of the 64 keys over the whole of R (mma.sync m16n8k16, float32 accumulation); the softmax's maxima and sums go
// through shared memory, P as bfloat16 too.  Sums: every warp takes a quarter of R over all 64 keys, the latents
// read as the B operand through a transposing ldmatrix, so each latent is fetched once for both products.
// ---------------------------------------------------------------------------------------------------------------
#define LM_KEYS 64
#define LM_ROWS 16
#define LM_PAD 8

__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_cp_async16(void* dst, const void* src, int src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d), "l"(src), "r"(src_bytes) : "memory");
}

// NT: n-tiles of 8 columns per warp in the second product, R = 32 * NT.  TT: tokens per block.  TT = 1: a block per
// row (blockIdx.x), any slices.  TT = 2: a block per tile of up to two tokens of one request, named by a tile list
// (tile_req[i] < 0: no tile); the two tokens' queries meet every tile of latents together, so a prompt's latents
// cross from L2 half as often and every B operand serves twice as many products.  One slice then.
template <int NT, int TT>
__global__ void __launch_bounds__(128)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long q_row, long q_head,
                            const __nv_bfloat16* __restrict__ plane, const int* __restrict__ block_table, int max_pages,
                            int page_size, int n_pages, const int* __restrict__ row_request,
                            const int* __restrict__ positions, const int* __restrict__ tile_req,
                            const int* __restrict__ tile_row0, const int* __restrict__ q_start, int n_heads, float scale,
                            int window, int n_slices, __nv_bfloat16* __restrict__ out, long o_row, long o_head,
                            float* __restrict__ ws_acc, float* __restrict__ ws_ml) {
    constexpr int R = 32 * NT, LDC = R + LM_PAD, LDP = LM_KEYS + LM_PAD, MR = TT * LM_ROWS;
    extern __shared__ __align__(16) unsigned char lm_smem[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);          // [TT * 16][LDC]
    __nv_bfloat16* c_s = q_s + MR * LDC;                                     // [64][LDC]
    __nv_bfloat16* p_s = c_s + LM_KEYS * LDC;                                // [TT * 16][LDP]
    float* pmax = reinterpret_cast<float*>(p_s + MR * LDP);                  // [4][TT * 16]
    float* psum = pmax + 4 * MR;                                             // [4][TT * 16]
    ib_grid_dependency_sync();
    const int slice = blockIdx.z, head0 = blockIdx.y * LM_ROWS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int row, req, n_tok = 1;
    if (TT == 1) {
        row = blockIdx.x;
        req = row_request[row];
    } else {
        req = tile_req[blockIdx.x];
        if (req < 0) return;                      // a place of the list without a tile (the whole block leaves)
        row = tile_row0[blockIdx.x];
        n_tok = min(TT, q_start[req + 1] - row);
    }
    const int pos0 = positions[row];              // the tokens of a tile stand at pos0, pos0 + 1, ...
    const int pos_last = pos0 + n_tok - 1;
    const int lo0 = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int* bt = block_table + (long)req * max_pages;
    const int first = (lo0 / LM_KEYS) * LM_KEYS;
    const int n_tiles = (pos_last - first) / LM_KEYS + 1;
    const int per_slice = (n_tiles + n_slices - 1) / n_slices;
    const int t0 = slice * per_slice, t1 = min(n_tiles, t0 + per_slice);

    // the queries of the group's heads (rows of heads and tokens that do not exist are zeros)
    for (int i = threadIdx.x; i < MR * (R / 8); i += blockDim.x) {
        const int m = i / (R / 8), ch = i % (R / 8);
        const int tok = m / LM_ROWS, h = head0 + m % LM_ROWS;
        const bool ok = h < n_heads && tok < n_tok;
        const __nv_bfloat16* src = q + (long)(row + (ok ? tok : 0)) * q_row + (long)min(h, n_heads - 1) * q_head + ch * 8;
        lm_cp_async16(q_s + m * LDC + ch * 8, src, ok ? 16 : 0);
    }
    // two threads per key: the page is looked up once per key and tile, each thread copies half of the latent
    auto load_tile = [&](int t) {
        const int jj = threadIdx.x >> 1, half = threadIdx.x & 1;
        const int j = first + t * LM_KEYS + jj;
        const __nv_bfloat16* src = plane;
        int bytes = 0;
        if (j >= lo0 && j <= pos_last) {
            const int page = bt[j / page_size];
            if (page >= 0 && page < n_pages) {
                src = plane + ((long)page * page_size + (j % page_size)) * R;
                bytes = 16;
            }
        }
        __nv_bfloat16* dst = c_s + jj * LDC;
#pragma unroll
        for (int ch = half; ch < R / 8; ch += 2) lm_cp_async16(dst + ch * 8, bytes ? src + ch * 8 : src, bytes);
    };
    if (t0 < t1) load_tile(t0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    float o[TT][NT][4];
    float m_run[TT][2], l_run[TT][2];                 // rows lane/4 and lane/4 + 8 of every token
#pragma unroll
    for (int tk = 0; tk < TT; ++tk) {
#pragma unroll
        for (int i = 0; i < NT; ++i) o[tk][i][0] = o[tk][i][1] = o[tk][i][2] = o[tk][i][3] = 0.0f;
        m_run[tk][0] = m_run[tk][1] = -INFINITY;
        l_run[tk][0] = l_run[tk][1] = 0.0f;
    }
    const int r_lo = lane >> 2, r_hi = r_lo + 8;

    for (int t = t0; t < t1; ++t) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const __nv_bfloat16* ct = c_s;
        // ---- scores of this warp's 16 keys, for every token -------------------------------------------------
        // (two sets of accumulators take turns, so that a product does not wait for the one before it)
        float sc[TT][2][4], sd[TT][2][4];
#pragma unroll
        for (int tk = 0; tk < TT; ++tk)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                sc[tk][i][0] = sc[tk][i][1] = sc[tk][i][2] = sc[tk][i][3] = 0.0f;
                sd[tk][i][0] = sd[tk][i][1] = sd[tk][i][2] = sd[tk][i][3] = 0.0f;
            }
#pragma unroll
        for (int ks = 0; ks < R / 16; ++ks) {
            uint32_t b0, b1, b2, b3;
            lm_ldmatrix_x4(b0, b1, b2, b3, ct + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * LDC + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int tk = 0; tk < TT; ++tk) {
                uint32_t a0, a1, a2, a3;
                lm_ldmatrix_x4(a0, a1, a2, a3, q_s + (tk * LM_ROWS + (lane & 15)) * LDC + ks * 16 + (lane >> 4) * 8);
                if (ks & 1) {
                    lm_mma(sd[tk][0], a0, a1, a2, a3, b0, b1);
                    lm_mma(sd[tk][1], a0, a1, a2, a3, b2, b3);
                } else {
                    lm_mma(sc[tk][0], a0, a1, a2, a3, b0, b1);
                    lm_mma(sc[tk][1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        const int j_base = first + t * LM_KEYS + warp * 16 + 2 * (lane & 3);
#pragma unroll
        for (int tk = 0; tk < TT; ++tk) {
            const int lo = lo0 + (window > 0 && pos0 + tk - window + 1 > 0 ? (pos0 + tk - window + 1) - lo0 : 0);
            const int hi = tk < n_tok ? pos0 + tk : -1;             // a token that does not exist sees nothing
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int j = j_base + i * 8 + (c & 1);
                    const float v = (j >= lo && j <= hi) ? (sc[tk][i][c] + sd[tk][i][c]) * scale : -INFINITY;
                    sc[tk][i][c] = v;
                    mx[c >> 1] = fmaxf(mx[c >> 1], v);
                }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 1));
                mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 2));
            }
            if ((lane & 3) == 0) {
                pmax[warp * MR + tk * LM_ROWS + r_lo] = mx[0];
                pmax[warp * MR + tk * LM_ROWS + r_hi] = mx[1];
            }
        }
        __syncthreads();
        float corr[TT][2];
#pragma unroll
        for (int tk = 0; tk < TT; ++tk) {
            float m_new[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int rr = tk * LM_ROWS + (k ? r_hi : r_lo);
                const float tm = fmaxf(fmaxf(pmax[rr], pmax[MR + rr]), fmaxf(pmax[2 * MR + rr], pmax[3 * MR + rr]));
                m_new[k] = fmaxf(m_run[tk][k], tm);
                corr[tk][k] = (m_run[tk][k] == -INFINITY) ? 0.0f : expf(m_run[tk][k] - m_new[k]);
                m_run[tk][k] = m_new[k];
            }
            float sm[2] = {0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float p[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    p[c] = (sc[tk][i][c] == -INFINITY) ? 0.0f : expf(sc[tk][i][c] - m_new[c >> 1]);
                    sm[c >> 1] += p[c];
                }
                const int col = warp * 16 + i * 8 + 2 * (lane & 3);
                *reinterpret_cast<__nv_bfloat162*>(p_s + (tk * LM_ROWS + r_lo) * LDP + col) = __floats2bfloat162_rn(p[0], p[1]);
                *reinterpret_cast<__nv_bfloat162*>(p_s + (tk * LM_ROWS + r_hi) * LDP + col) = __floats2bfloat162_rn(p[2], p[3]);
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                sm[k] += __shfl_xor_sync(0xffffffffu, sm[k], 1);
                sm[k] += __shfl_xor_sync(0xffffffffu, sm[k], 2);
            }
            if ((lane & 3) == 0) {
                psum[warp * MR + tk * LM_ROWS + r_lo] = sm[0];
                psum[warp * MR + tk * LM_ROWS + r_hi] = sm[1];
            }
        }
        __syncthreads();
#pragma unroll
        for (int tk = 0; tk < TT; ++tk) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int rr = tk * LM_ROWS + (k ? r_hi : r_lo);
                l_run[tk][k] = l_run[tk][k] * corr[tk][k] + ((psum[rr] + psum[MR + rr]) + (psum[2 * MR + rr] + psum[3 * MR + rr]));
            }
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                o[tk][i][0] *= corr[tk][0]; o[tk][i][1] *= corr[tk][0];
                o[tk][i][2] *= corr[tk][1]; o[tk][i][3] *= corr[tk][1];
            }
        }
        // ---- this warp's quarter of the sums over all 64 keys, for every token -------------------------------
#pragma unroll
        for (int kk = 0; kk < LM_KEYS / 16; ++kk) {
            uint32_t a[TT][4];
#pragma unroll
            for (int tk = 0; tk < TT; ++tk)
                lm_ldmatrix_x4(a[tk][0], a[tk][1], a[tk][2], a[tk][3], p_s + (tk * LM_ROWS + (lane & 15)) * LDP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int i = 0; i < NT; i += 2) {
                uint32_t b0, b1, b2, b3;
                lm_ldmatrix_x4_trans(b0, b1, b2, b3, ct + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDC + warp * (R / 4) + i * 8 + (lane >> 4) * 8);
#pragma unroll
                for (int tk = 0; tk < TT; ++tk) {
                    lm_mma(o[tk][i], a[tk][0], a[tk][1], a[tk][2], a[tk][3], b0, b1);
                    if (i + 1 < NT) lm_mma(o[tk][i + 1], a[tk][0], a[tk][1], a[tk][2], a[tk][3], b2, b3);   // an odd last tile: the other half read padding
                }
            }
        }
        __syncthreads();      // the buffer, P and the maxima are free for the next tile
        if (t + 1 < t1) load_tile(t + 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // ---- out ------------------------------------------------------------------------------------------------
#pragma unroll
    for (int tk = 0; tk < TT; ++tk) {
        if (tk >= n_tok) continue;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int h = head0 + (k ? r_hi : r_lo);
            if (h >= n_heads) continue;
            if (n_slices == 1) {
                const float inv = l_run[tk][k] > 0.0f ? 1.0f / l_run[tk][k] : 0.0f;
                __nv_bfloat16* dst = out + (long)(row + tk) * o_row + (long)h * o_head + warp * (R / 4) + 2 * (lane & 3);
#pragma unroll
                for (int i = 0; i < NT; ++i)
                    *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) =
                        __floats2bfloat162_rn(o[tk][i][2 * k] * inv, o[tk][i][2 * k + 1] * inv);
            } else {
                const long item = ((long)(row + tk) * n_heads + h) * n_slices + slice;
                float* dst = ws_acc + item * R + warp * (R / 4) + 2 * (lane & 3);
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    dst[i * 8] = o[tk][i][2 * k];
                    dst[i * 8 + 1] = o[tk][i][2 * k + 1];
                }
                if (warp == 0 && (lane & 3) == 0) {
                    ws_ml[item * 2] = m_run[tk][k];
                    ws_ml[item * 2 + 1] = l_run[tk][k];
                }
            }
        }
    }
}

static IbDeviceSet latent_mma_smem_set[2][17];

template <int NT, int TT>
static int launch_latent_mma(const void* q, long q_row, long q_head, const void* plane, const int* block_table,
                             int max_pages, int page_size, int n_pages, const int* row_request, const int* positions,
                             const int* tile_req, const int* tile_row0, const int* q_start, int n_blocks, int n_heads,
                             float scale, int window, int n_slices, void* out, long o_row, long o_head, float* ws_acc,
                             float* ws_ml, cudaStream_t stream) {
    constexpr int R = 32 * NT, LDC = R + LM_PAD, LDP = LM_KEYS + LM_PAD, MR = TT * LM_ROWS;
    const size_t smem = (size_t)(MR * LDC + LM_KEYS * LDC + MR * LDP) * 2 + 8 * MR * sizeof(float);
    if (smem > 48 * 1024) {
        const int e = ib_allow_dynamic_smem(latent_mma_smem_set[TT - 1][NT], latent_attention_mma_kernel<NT, TT>, smem);
        if (e != IB_OK) return e;
    }
    const dim3 grid(n_blocks, (n_heads + LM_ROWS - 1) / LM_ROWS, n_slices);
    ib_launch(latent_attention_mma_kernel<NT, TT>, grid, 128, smem, stream, (const __nv_bfloat16*)q, q_row, q_head,
              (const __nv_bfloat16*)plane, block_table, max_pages, page_size, n_pages, row_request, positions, tile_req,
              tile_row0, q_start, n_heads, scale, window, n_slices, (__nv_bfloat16*)out, o_row, o_head, ws_acc, ws_ml);
    return ib_launch_status();
}
#endif  // IB_ACT_BF16

static IbDeviceSet latent_smem_set[2][5];

template <typename QT, int RPL>
static int launch_latent(IbDeviceSet& set, const void* q, long q_row, long q_head, const void* plane,
                         const int* block_table, int max_pages, int page_size, int n_pages, const int* row_request,
                         const int* positions, int n_rows, int n_heads, int R, float scale, int window, int n_slices,
                         void* out, long o_row, long o_head, float* ws_acc, float* ws_ml, cudaStream_t stream) {
    const size_t smem = ((size_t)LA_KEYS * (R + 1) + (size_t)LA_HEADS * R) * sizeof(float);
    // the most that this form of the kernel can ask for: the permission is given once per device
    const size_t smem_most = ((size_t)LA_KEYS * (32 * RPL + 1) + (size_t)LA_HEADS * 32 * RPL) * sizeof(float);
    if (smem_most > 48 * 1024) {
        const int e = ib_allow_dynamic_smem(set, latent_attention_kernel<QT, RPL>, smem_most);
        if (e != IB_OK) return e;
    }
    const dim3 grid(n_rows, (n_heads + LA_HEADS - 1) / LA_HEADS, n_slices);
    ib_launch(latent_attention_kernel<QT, RPL>, grid, 32 * LA_WARPS, smem, stream, (const QT*)q, q_row, q_head,
              (const act_t*)plane, block_table, max_pages, page_size, n_pages, row_request, positions, n_heads, R, scale,
              window, n_slices, (act_t*)out, o_row, o_head, ws_acc, ws_ml);
    return ib_launch_status();
}

// q: element (row, h, e) at q[row * q_row + h * q_head + e], float (q_is_f32) or act_t; out likewise, act_t.
// plane [n_pages, page_size, R] act_t.  n_slices > 1 needs ws_acc [rows * heads * n_slices * R] and
// ws_ml [rows * heads * n_slices * 2] floats.  tile_req, tile_row0 [n_tiles] and q_start (or null): the step's rows
// cut into tiles of up to two tokens of one request each; the tensor-core form then takes two tokens per block.
IB_EXPORT int ib_latent_attention(const void* q, int q_is_f32, long q_row, long q_head, const void* plane,
                                  const int* block_table, int max_pages, int page_size, int n_pages,
                                  const int* row_request, const int* positions, int n_rows, int n_heads, int R,
                                  float scale, int window, int n_slices, void* out, long o_row, long o_head,
                                  float* ws_acc, float* ws_ml, const int* tile_req, const int* tile_row0,
                                  const int* q_start, int n_tiles, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (n_heads <= 0 || R <= 0 || page_size <= 0 || max_pages <= 0 || n_slices <= 0 || n_slices > 64 ||
        (n_slices > 1 && (ws_acc == nullptr || ws_ml == nullptr)))
        return IB_ERR_ARGUMENT;
    if (R > 512) return IB_ERR_UNSUPPORTED;
    int e = IB_OK;
#if IB_ACT_BF16
    // bfloat16 queries and latents of a multiple of 32 numbers: the tensor cores
    if (!q_is_f32 && R % 32 == 0 && page_size > 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)plane % 16) == 0) {
        // a list of tiles of up to two tokens (prompt portions, one slice): two tokens per block
        const bool pairs = tile_req != nullptr && tile_row0 != nullptr && q_start != nullptr && n_tiles > 0 && n_slices == 1;
        switch (R / 32) {
#define IB_LATM(NT)                                                                                                  \
        case NT:                                                                                                     \
            e = pairs ? launch_latent_mma<NT, 2>(q, q_row, q_head, plane, block_table, max_pages, page_size, n_pages, \
                                                 row_request, positions, tile_req, tile_row0, q_start, n_tiles,      \
                                                 n_heads, scale, window, 1, out, o_row, o_head, ws_acc, ws_ml, stream) \
                      : launch_latent_mma<NT, 1>(q, q_row, q_head, plane, block_table, max_pages, page_size, n_pages, \
                                                 row_request, positions, nullptr, nullptr, nullptr, n_rows, n_heads, \
                                                 scale, window, n_slices, out, o_row, o_head, ws_acc, ws_ml, stream); \
            break;
            IB_LATM(1) IB_LATM(2) IB_LATM(3) IB_LATM(4) IB_LATM(5) IB_LATM(6) IB_LATM(7) IB_LATM(8) IB_LATM(9)
            IB_LATM(10) IB_LATM(11) IB_LATM(12) IB_LATM(13) IB_LATM(14) IB_LATM(15) IB_LATM(16)
#undef IB_LATM
            default: e = IB_ERR_UNSUPPORTED;
        }
        if (e != IB_ERR_UNSUPPORTED) {
            if (e != IB_OK || n_slices == 1) return e;
            const int jw = 4;
            const long n_items = (long)n_rows * n_heads;
            ib_launch(latent_attention_join_kernel, (unsigned)((n_items + jw - 1) / jw), 32 * jw, 0, stream, ws_acc, ws_ml,
                      n_rows, n_heads, R, n_slices, (act_t*)out, o_row, o_head);
            return ib_launch_status();
        }
        e = IB_OK;
    }
#endif
#define IB_LAT(QT, QI, RPL, SI)                                                                                   \
    e = launch_latent<QT, RPL>(latent_smem_set[QI][SI], q, q_row, q_head, plane, block_table, max_pages, page_size, \
                               n_pages, row_request, positions, n_rows, n_heads, R, scale, window, n_slices, out,  \
                               o_row, o_head, ws_acc, ws_ml, stream)
#define IB_LAT_R(QT, QI)                                                                                          \
    do {                                                                                                          \
        if (R <= 32) IB_LAT(QT, QI, 1, 0); else if (R <= 64) IB_LAT(QT, QI, 2, 1);                                \
        else if (R <= 128) IB_LAT(QT, QI, 4, 2); else if (R <= 256) IB_LAT(QT, QI, 8, 3);                         \
        else IB_LAT(QT, QI, 16, 4);                                                                               \
    } while (0)
    if (q_is_f32) IB_LAT_R(float, 0); else IB_LAT_R(act_t, 1);
#undef IB_LAT_R
#undef IB_LAT
    if (e != IB_OK || n_slices == 1) return e;
    const int warps = 4;
    const long items = (long)n_rows * n_heads;
    ib_launch(latent_attention_join_kernel, (unsigned)((items + warps - 1) / warps), 32 * warps, 0, stream, ws_acc, ws_ml,
              n_rows, n_heads, R, n_slices, (act_t*)out, o_row, o_head);
    return ib_launch_status();
}
