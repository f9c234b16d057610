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

// Joins the slices of one (row, head): a warp each, slices in ascending order.
__global__ void latent_attention_join_kernel(const float* __restrict__ ws_acc, const float* __restrict__ ws_ml,
                                             int n_rows, int n_heads, int R, int n_slices, act_t* __restrict__ out,
                                             long o_row, long o_head) {
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)n_rows * n_heads) return;
    const int row = (int)(item / n_heads), h = (int)(item % n_heads);
    float m = -INFINITY;
    for (int s = 0; s < n_slices; ++s) m = fmaxf(m, ws_ml[(item * n_slices + s) * 2]);
    float l = 0.0f;
    for (int s = 0; s < n_slices; ++s) {
        const float ms = ws_ml[(item * n_slices + s) * 2];
        if (ms != -INFINITY) l += ws_ml[(item * n_slices + s) * 2 + 1] * expf(ms - m);
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    act_t* dst = out + (long)row * o_row + (long)h * o_head;
    for (int e = lane; e < R; e += 32) {
        float v = 0.0f;
        for (int s = 0; s < n_slices; ++s) {
            const float ms = ws_ml[(item * n_slices + s) * 2];
            if (ms != -INFINITY) v = fmaf(ws_acc[(item * n_slices + s) * R + e], expf(ms - m), v);
        }
        dst[e] = ib_from_float<act_t>(v * inv);
    }
}

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
// ws_ml [rows * heads * n_slices * 2] floats.
IB_EXPORT int ib_latent_attention(const void* q, int q_is_f32, long q_row, long q_head, const void* plane,
                                  const int* block_table, int max_pages, int page_size, int n_pages,
                                  const int* row_request, const int* positions, int n_rows, int n_heads, int R,
                                  float scale, int window, int n_slices, void* out, long o_row, long o_head,
                                  float* ws_acc, float* ws_ml, cudaStream_t stream) {
    if (n_rows <= 0) return IB_OK;
    if (n_heads <= 0 || R <= 0 || page_size <= 0 || max_pages <= 0 || n_slices <= 0 || n_slices > 65535 ||
        (n_slices > 1 && (ws_acc == nullptr || ws_ml == nullptr)))
        return IB_ERR_ARGUMENT;
    if (R > 512) return IB_ERR_UNSUPPORTED;
    int e = IB_OK;
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
