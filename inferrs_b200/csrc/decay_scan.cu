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
// Work split: a block owns COLS columns of S for one (request, head): 32 (lane l owns column l, warp w the rows
// 16 w .. 16 w + 15 of S, in registers), or 16 where a step has too few (request, head, 32 columns) to give every SM
// a block (the two halves of a warp then own the same 16 columns and eight rows each).  Tokens go in chunks of 16
// through shared memory, two buffers: the next chunk's q, k, v, keep and take are on their way (cp.async, nothing
// waits in registers) while the chunk before is walked.  Per token a lane does its rows' multiply-adds for the
// update and as many for the product with q; the warps' shares of the product are summed through shared memory
// once per chunk, in a fixed order.  A step of single tokens takes chunks of one.
//
// State of one slot: S as [H, D, E] floats (E contiguous) from the slot's first float on.
#include "common.cuh"

#define DS_ROWS 16     // rows of S per warp

__device__ __forceinline__ void ds_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ds_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// VEC: 4 where q, k and v rows can be fetched sixteen bytes at a time (the host checks sizes and alignment), else 1.
template <int CH, int COLS, int VEC>
__global__ void decay_scan_kernel(const float* __restrict__ x, long ld, int q_col, int k_col, int v_col, int G,
                                  const float* __restrict__ keep, long keep_ld, const float* __restrict__ take,
                                  long take_ld, const float* __restrict__ skip, float* __restrict__ state,
                                  long slot_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                                  float* __restrict__ out, int H, int D, int E) {
    extern __shared__ __align__(16) float smem[];
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    constexpr int HALVES = 32 / COLS, RL = DS_ROWS / HALVES;      // rows of S per lane
    const int Dp = n_warps * DS_ROWS;                             // D rounded up: the rows beyond D hold zeros
    const int col = lane % COLS, half_w = lane / COLS, n_units = n_warps * HALVES;
    const int h = blockIdx.y, r = blockIdx.z, e0 = blockIdx.x * COLS, dl = warp * DS_ROWS + half_w * RL;
    const int g = h / (H / G);
    const int row0 = q_start[r], row1 = q_start[r + 1];
    if (row1 <= row0) return;                                     // the whole block leaves
    // q [CH][Dp], k [CH][Dp], v [CH][COLS], keep [CH], take [CH]; the second buffer starts on a 16-byte boundary too
    const int buf_floats = (2 * CH * Dp + CH * COLS + 2 * CH + 3) & ~3;
    float* part = smem + 2 * buf_floats;                          // [CH][n_units][COLS]
    // what no copy writes stays as it is set here: zeros in the rows beyond D and the columns beyond E, ones where
    // there is no take
    for (int i = threadIdx.x; i < 2 * buf_floats; i += blockDim.x) {
        const int j = i % buf_floats;
        smem[i] = (j >= 2 * CH * Dp + CH * COLS + CH && j < 2 * CH * Dp + CH * COLS + 2 * CH) ? 1.0f : 0.0f;
    }
    __syncthreads();

    float* st = state + (long)slots[r] * slot_stride + (long)h * D * E;
    const bool col_ok = e0 + col < E;
    float S[RL];
#pragma unroll
    for (int i = 0; i < RL; ++i) S[i] = (col_ok && dl + i < D) ? st[(long)(dl + i) * E + e0 + col] : 0.0f;
    const float skip_h = skip ? skip[h] : 0.0f;
    const int e_n = min(COLS, E - e0);                            // this block's columns that exist

    auto fetch = [&](int c0, int buf) {
        const int nc = min(CH, row1 - c0);
        float* q_s = smem + buf * buf_floats;
        float* k_s = q_s + CH * Dp;
        float* v_s = k_s + CH * Dp;
        float* g_s = v_s + CH * COLS;
        if (VEC == 4) {
            const int d4 = D >> 2;
            for (int idx = threadIdx.x; idx < nc * d4; idx += blockDim.x) {
                const int t = idx / d4, d = (idx - t * d4) << 2;
                const float* xr = x + (long)(c0 + t) * ld + g * D + d;
                ds_copy16(q_s + t * Dp + d, xr + q_col);
                ds_copy16(k_s + t * Dp + d, xr + k_col);
            }
            const int e4 = e_n >> 2;
            for (int idx = threadIdx.x; idx < nc * e4; idx += blockDim.x) {
                const int t = idx / e4, e = (idx - t * e4) << 2;
                ds_copy16(v_s + t * COLS + e, x + (long)(c0 + t) * ld + v_col + h * E + e0 + e);
            }
        } else {
            for (int idx = threadIdx.x; idx < nc * D; idx += blockDim.x) {
                const int t = idx / D, d = idx - t * D;
                const float* xr = x + (long)(c0 + t) * ld + g * D + d;
                ds_copy4(q_s + t * Dp + d, xr + q_col);
                ds_copy4(k_s + t * Dp + d, xr + k_col);
            }
            for (int idx = threadIdx.x; idx < nc * e_n; idx += blockDim.x) {
                const int t = idx / e_n, e = idx - t * e_n;
                ds_copy4(v_s + t * COLS + e, x + (long)(c0 + t) * ld + v_col + h * E + e0 + e);
            }
        }
        if (threadIdx.x < nc) {
            ds_copy4(g_s + threadIdx.x, keep + (long)(c0 + threadIdx.x) * keep_ld + h);
            if (take) ds_copy4(g_s + CH + threadIdx.x, take + (long)(c0 + threadIdx.x) * take_ld + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(row0, 0);

    int buf = 0;
    for (int c0 = row0; c0 < row1; c0 += CH, buf ^= 1) {
        const int nc = min(CH, row1 - c0);
        if (c0 + CH < row1) {
            fetch(c0 + CH, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* q_s = smem + buf * buf_floats;
        const float* k_s = q_s + CH * Dp;
        const float* v_s = k_s + CH * Dp;
        const float* g_s = v_s + CH * COLS;
        // ---- the tokens, one after the other ------------------------------------------------------------------
        for (int t = 0; t < nc; ++t) {
            const float kp = g_s[t];
            const float vt = v_s[t * COLS + col] * g_s[CH + t];
            const float4* q4 = reinterpret_cast<const float4*>(q_s + t * Dp + dl);
            const float4* k4 = reinterpret_cast<const float4*>(k_s + t * Dp + dl);
            float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
#pragma unroll
            for (int i = 0; i < RL / 4; ++i) {
                const float4 q = q4[i], k = k4[i];
                S[4 * i + 0] = fmaf(kp, S[4 * i + 0], k.x * vt); acc0 = fmaf(S[4 * i + 0], q.x, acc0);
                S[4 * i + 1] = fmaf(kp, S[4 * i + 1], k.y * vt); acc1 = fmaf(S[4 * i + 1], q.y, acc1);
                S[4 * i + 2] = fmaf(kp, S[4 * i + 2], k.z * vt); acc2 = fmaf(S[4 * i + 2], q.z, acc2);
                S[4 * i + 3] = fmaf(kp, S[4 * i + 3], k.w * vt); acc3 = fmaf(S[4 * i + 3], q.w, acc3);
            }
            part[(t * n_units + warp * HALVES + half_w) * COLS + col] = (acc0 + acc1) + (acc2 + acc3);
        }
        __syncthreads();
        // ---- the warps' shares of every token's product, summed in a fixed order ------------------------------
        for (int idx = threadIdx.x; idx < nc * COLS; idx += blockDim.x) {
            const int t = idx / COLS, e = idx - t * COLS;
            float o = 0.0f;
            for (int u = 0; u < n_units; ++u) o += part[(t * n_units + u) * COLS + e];
            if (e0 + e < E) out[((long)(c0 + t) * H + h) * E + e0 + e] = fmaf(skip_h, v_s[idx], o);
        }
        __syncthreads();       // before the next turn's copies overwrite this buffer
    }
#pragma unroll
    for (int i = 0; i < RL; ++i)
        if (col_ok && dl + i < D) st[(long)(dl + i) * E + e0 + col] = S[i];
}

static IbDeviceSet decay_scan_smem_set[8];

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
    if (D > 256 || H > 65535 || n_requests > 65535) return IB_ERR_UNSUPPORTED;   // sixteen warps of sixteen rows
    const int n_warps = (D + DS_ROWS - 1) / DS_ROWS;
    const int ch = max_rows == 1 ? 1 : 16;
    // 16 columns per block where 32 would leave most SMs without a block (prompt portions of a few requests)
    const int cols = (ch > 1 && E % 16 == 0 && (long)((E + 31) / 32) * H * n_requests < 120) ? 16 : 32;
    const dim3 grid((E + cols - 1) / cols, H, n_requests);
    // sixteen bytes at a time where every row, slice and head starts on such a boundary
    const bool vec = ((uintptr_t)x % 16) == 0 && (ld % 4) == 0 && (q_col % 4) == 0 && (k_col % 4) == 0 &&
                     (v_col % 4) == 0 && (D % 4) == 0 && (E % 4) == 0;
    const int units = n_warps * (32 / cols);
    const size_t smem = (size_t)(2 * ((2 * ch * n_warps * DS_ROWS + ch * cols + 2 * ch + 3) & ~3) + ch * units * cols) * sizeof(float);
#define IB_DSCAN(CH, COLS, VEC, SET)                                                                               \
    do {                                                                                                           \
        if (smem > 48 * 1024) {                                                                                    \
            const int e = ib_allow_dynamic_smem(decay_scan_smem_set[SET], decay_scan_kernel<CH, COLS, VEC>, 224 * 1024); \
            if (e != IB_OK) return e;                                                                              \
        }                                                                                                          \
        ib_launch(decay_scan_kernel<CH, COLS, VEC>, grid, 32 * n_warps, smem, stream, x, ld, q_col, k_col, v_col,  \
                  G, keep, keep_ld, take, take_ld, skip, state, slot_stride, q_start, slots, out, H, D, E);        \
    } while (0)
    if (ch == 1) { if (vec) IB_DSCAN(1, 32, 4, 0); else IB_DSCAN(1, 32, 1, 1); }
    else if (cols == 16) { if (vec) IB_DSCAN(16, 16, 4, 2); else IB_DSCAN(16, 16, 1, 3); }
    else { if (vec) IB_DSCAN(16, 32, 4, 4); else IB_DSCAN(16, 32, 1, 5); }
#undef IB_DSCAN
    return ib_launch_status();
}
