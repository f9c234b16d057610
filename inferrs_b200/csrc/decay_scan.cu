// A matrix state per head with a scalar decay, carried from token to token:
//
//     S_t = keep_t S_{t-1} + take_t k_t v_t^T          S is [D, E] per head
//     o_t = S_t^T q_t + skip v_t
//
// keep and take are one number per (token, head): a constant per head for a linear attention with a fixed decay
// (take absent: 1), exp(-exp(A) dt) and dt for a state-space mixer.  q and k may be shared by the heads of a
// group (head h reads group h / (H / G)); skip is one number per head (absent: 0).
//
// Everything is float in both builds: the kernels before this one hand in q, k and v as float rows (rotated,
// scaled, convolved as their mixer wants), and the state lives in float.  A request's rows are walked in order,
// one token after the other, so a result does not depend on how the prompt was cut into steps or on what else the
// step holds.
//
// Work split: a block owns 32 columns of S for one (request, head); lane l owns column l, warp w the rows
// 16 w .. 16 w + 15 of S, in registers.  Tokens go in chunks of 16 through shared memory; per token a lane does 16
// multiply-adds for the update and 16 for the product with q, and the warps' shares of the product are summed
// through shared memory once per chunk.  A step of single tokens takes chunks of one.
//
// State of one slot: S as [H, D, E] floats (E contiguous) from the slot's first float on.
#include "common.cuh"

#define DS_ROWS 16     // rows of S per warp
#define DS_COLS 32     // columns of S per block

template <int CH>
__global__ void decay_scan_kernel(const float* __restrict__ x, long ld, int q_col, int k_col, int v_col, int G,
                                  const float* __restrict__ keep, long keep_ld, const float* __restrict__ take,
                                  long take_ld, const float* __restrict__ skip, float* __restrict__ state,
                                  long slot_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                                  float* __restrict__ out, int H, int D, int E) {
    extern __shared__ __align__(16) float smem[];
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int Dp = n_warps * DS_ROWS;                    // D rounded up: the rows beyond D hold zeros
    const int h = blockIdx.y, r = blockIdx.z, e0 = blockIdx.x * DS_COLS, d0 = warp * DS_ROWS;
    const int g = h / (H / G);
    const int row0 = q_start[r], row1 = q_start[r + 1];
    if (row1 <= row0) return;                            // the whole block leaves
    float* q_s = smem;                                   // [CH][Dp]
    float* k_s = q_s + CH * Dp;                          // [CH][Dp]
    float* v_s = k_s + CH * Dp;                          // [CH][DS_COLS]
    float* g_s = v_s + CH * DS_COLS;                     // [2][CH]: keep, take
    float* part = g_s + 2 * CH;                          // [CH][n_warps][DS_COLS]

    float* st = state + (long)slots[r] * slot_stride + (long)h * D * E;
    const bool col_ok = e0 + lane < E;
    float S[DS_ROWS];
#pragma unroll
    for (int i = 0; i < DS_ROWS; ++i) S[i] = (col_ok && d0 + i < D) ? st[(long)(d0 + i) * E + e0 + lane] : 0.0f;
    const float skip_h = skip ? skip[h] : 0.0f;

    for (int c0 = row0; c0 < row1; c0 += CH) {
        const int nc = min(CH, row1 - c0);
        for (int idx = threadIdx.x; idx < nc * Dp; idx += blockDim.x) {
            const int t = idx / Dp, d = idx - t * Dp;
            const float* xr = x + (long)(c0 + t) * ld;
            q_s[idx] = d < D ? xr[q_col + g * D + d] : 0.0f;
            k_s[idx] = d < D ? xr[k_col + g * D + d] : 0.0f;
        }
        for (int idx = threadIdx.x; idx < nc * DS_COLS; idx += blockDim.x) {
            const int t = idx / DS_COLS, e = idx - t * DS_COLS;
            v_s[idx] = e0 + e < E ? x[(long)(c0 + t) * ld + v_col + h * E + e0 + e] : 0.0f;
        }
        if (threadIdx.x < nc) {
            g_s[threadIdx.x] = keep[(long)(c0 + threadIdx.x) * keep_ld + h];
            g_s[CH + threadIdx.x] = take ? take[(long)(c0 + threadIdx.x) * take_ld + h] : 1.0f;
        }
        __syncthreads();
        // ---- the tokens, one after the other ------------------------------------------------------------------
        for (int t = 0; t < nc; ++t) {
            const float kp = g_s[t];
            const float vt = v_s[t * DS_COLS + lane] * g_s[CH + t];
            const float4* q4 = reinterpret_cast<const float4*>(q_s + t * Dp + d0);
            const float4* k4 = reinterpret_cast<const float4*>(k_s + t * Dp + d0);
            float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
#pragma unroll
            for (int i = 0; i < DS_ROWS / 4; ++i) {
                const float4 q = q4[i], k = k4[i];
                S[4 * i + 0] = fmaf(kp, S[4 * i + 0], k.x * vt); acc0 = fmaf(S[4 * i + 0], q.x, acc0);
                S[4 * i + 1] = fmaf(kp, S[4 * i + 1], k.y * vt); acc1 = fmaf(S[4 * i + 1], q.y, acc1);
                S[4 * i + 2] = fmaf(kp, S[4 * i + 2], k.z * vt); acc2 = fmaf(S[4 * i + 2], q.z, acc2);
                S[4 * i + 3] = fmaf(kp, S[4 * i + 3], k.w * vt); acc3 = fmaf(S[4 * i + 3], q.w, acc3);
            }
            part[(t * n_warps + warp) * DS_COLS + lane] = (acc0 + acc1) + (acc2 + acc3);
        }
        __syncthreads();
        // ---- the warps' shares of every token's product, summed in a fixed order ------------------------------
        for (int idx = threadIdx.x; idx < nc * DS_COLS; idx += blockDim.x) {
            const int t = idx / DS_COLS, e = idx - t * DS_COLS;
            float o = 0.0f;
            for (int w = 0; w < n_warps; ++w) o += part[(t * n_warps + w) * DS_COLS + e];
            if (e0 + e < E) out[((long)(c0 + t) * H + h) * E + e0 + e] = fmaf(skip_h, v_s[idx], o);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < DS_ROWS; ++i)
        if (col_ok && d0 + i < D) st[(long)(d0 + i) * E + e0 + lane] = S[i];
}

static IbDeviceSet decay_scan_smem_set[2];

// x [rows, ld] float holds q and k as [G, D] and v as [H, E] from columns q_col, k_col, v_col on.  keep [rows,
// keep_ld] (keep_ld 0: one row of H numbers for all tokens), take likewise or absent (1), skip [H] or absent (0).
// out [rows, H, E] float.  max_rows: the most rows that a request brings (1: the form for steps of single tokens).
IB_EXPORT int ib_decay_scan(const float* x, long ld, int q_col, int k_col, int v_col, int G, const float* keep,
                            long keep_ld, const float* take, long take_ld, const float* skip, float* state,
                            long slot_stride, const int* q_start, const int* slots, int n_requests, float* out, int H,
                            int D, int E, int max_rows, cudaStream_t stream) {
    if (n_requests <= 0) return IB_OK;
    if (H <= 0 || D <= 0 || E <= 0 || G <= 0 || H % G || x == nullptr || keep == nullptr || state == nullptr ||
        out == nullptr || slot_stride < (long)H * D * E)
        return IB_ERR_ARGUMENT;
    if (D > 512 || H > 65535 || n_requests > 65535) return IB_ERR_UNSUPPORTED;
    const int n_warps = (D + DS_ROWS - 1) / DS_ROWS;
    const dim3 grid((E + DS_COLS - 1) / DS_COLS, H, n_requests);
    const int ch = max_rows == 1 ? 1 : 16;
    const size_t smem = (size_t)(2 * ch * n_warps * DS_ROWS + ch * DS_COLS + 2 * ch + ch * n_warps * DS_COLS) * sizeof(float);
#define IB_DSCAN(CH, SET)                                                                                          \
    do {                                                                                                           \
        if (smem > 48 * 1024) {                                                                                    \
            const int e = ib_allow_dynamic_smem(decay_scan_smem_set[SET], decay_scan_kernel<CH>, 160 * 1024);      \
            if (e != IB_OK) return e;                                                                              \
        }                                                                                                          \
        ib_launch(decay_scan_kernel<CH>, grid, 32 * n_warps, smem, stream, x, ld, q_col, k_col, v_col, G, keep,    \
                  keep_ld, take, take_ld, skip, state, slot_stride, q_start, slots, out, H, D, E);                 \
    } while (0)
    if (ch == 1) IB_DSCAN(1, 0); else IB_DSCAN(16, 1);
#undef IB_DSCAN
    return ib_launch_status();
}
