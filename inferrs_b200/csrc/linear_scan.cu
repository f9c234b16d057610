// Mixers with a matrix state per head that is carried from token to token:
//
//   mode 0, a decay per key channel (gated linear attention):
//       S_t = diag(a_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t,   a_t = sigmoid(z_t + b)^(1/tau)
//   mode 1, scalar gates with a running maximum (the matrix memory of xLSTM):
//       i_t = cap tanh((p_t + b_i) / cap),   f_t = logsigmoid(cap tanh((r_t + b_f) / cap))
//       m_t = max(f_t + m_{t-1}, i_t)
//       S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T        (n_t the same with k_t alone)
//       o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// S is [D, E] per head (D key channels, E value channels).  The state, the gates and every sum are float in both
// builds; q, k and v come from a projection in act_t.  A request's rows are walked in order, one token after the
// other, so a result does not depend on how the prompt was cut into steps or on what else the step holds.
//
// Work split: a warp owns four columns of S for one (request, head); lane l owns the rows l, l + 32, ...  A token
// costs the warp its q, k and gate loads (fetched one token ahead), D * 4 / 32 multiply-adds per lane for the update
// and as many for the product with q, and one warp sum per column.  The warps of a block own neighbouring columns
// of the same head, so q, k and the gates are fetched from L1 after the first warp.
//
// State of one slot, float: S as [H, E, D] (D contiguous, so a warp's loads and stores are whole lines), then for
// mode 1 n as [H, D] and m as [H].
#include "common.cuh"

#define LS_WARPS 8
#define LS_COLS 4

__device__ __forceinline__ float ls_logsigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

template <int MODE, int NK>
__global__ void __launch_bounds__(32 * LS_WARPS)
linear_scan_kernel(const act_t* __restrict__ proj, long ld, int q_col, int k_col, int v_col,
                   const float* __restrict__ gates, long ld_gates, const float* __restrict__ gate_bias,
                   float gate_param, float q_scale, float* __restrict__ state, long slot_stride,
                   const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ out,
                   int H, int D, int E) {
    ib_grid_dependency_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, r = blockIdx.z;
    const int e0 = (blockIdx.x * LS_WARPS + warp) * LS_COLS;
    if (e0 >= E) return;                       // whole warps leave; only warp-level exchanges follow
    const int row0 = q_start[r], row1 = q_start[r + 1];
    if (row1 <= row0) return;
    float* st = state + (long)slots[r] * slot_stride;
    float* st_S = st + ((long)h * E + e0) * D;
    float* st_n = st + (long)H * E * D + (long)h * D;
    float* st_m = st + (long)H * E * D + (long)H * D + h;

    float S[NK][LS_COLS], nvec[NK];
    float m = 0.0f;
#pragma unroll
    for (int k = 0; k < NK; ++k) {
        const int d = lane + 32 * k;
#pragma unroll
        for (int c = 0; c < LS_COLS; ++c) S[k][c] = (d < D && e0 + c < E) ? st_S[(long)c * D + d] : 0.0f;
        nvec[k] = (MODE == 1 && d < D) ? st_n[d] : 0.0f;
    }
    if (MODE == 1) m = *st_m;

    float bias[NK];
    float b_i = 0.0f, b_f = 0.0f;
    if (MODE == 0) {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const int d = lane + 32 * k;
            bias[k] = d < D ? gate_bias[h * D + d] : 0.0f;
        }
    } else {
        b_i = gate_bias[h];
        b_f = gate_bias[H + h];
    }

    // one token's inputs, fetched a token ahead of their use
    float nq[NK], nk[NK], ng[NK] = {}, nv[LS_COLS], ngi = 0.0f, ngf = 0.0f;
    auto fetch = [&](int row) {
        const act_t* p = proj + (long)row * ld;
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            const int d = lane + 32 * k;
            const bool ok = d < D;
            nq[k] = ok ? ib_to_float(p[q_col + h * D + d]) : 0.0f;
            nk[k] = ok ? ib_to_float(p[k_col + h * D + d]) : 0.0f;
            if (MODE == 0) ng[k] = ok ? gates[(long)row * ld_gates + h * D + d] : 0.0f;
        }
#pragma unroll
        for (int c = 0; c < LS_COLS; ++c) nv[c] = (e0 + c < E) ? ib_to_float(p[v_col + h * E + e0 + c]) : 0.0f;
        if (MODE == 1) {
            ngi = gates[(long)row * ld_gates + h];
            ngf = gates[(long)row * ld_gates + H + h];
        }
    };
    fetch(row0);
    for (int row = row0; row < row1; ++row) {
        float q[NK], kk[NK], g[NK], v[LS_COLS];
#pragma unroll
        for (int k = 0; k < NK; ++k) { q[k] = nq[k] * q_scale; kk[k] = nk[k]; g[k] = ng[k]; }
#pragma unroll
        for (int c = 0; c < LS_COLS; ++c) v[c] = nv[c];
        const float gi = ngi, gf = ngf;
        if (row + 1 < row1) fetch(row + 1);

        float o[LS_COLS];
#pragma unroll
        for (int c = 0; c < LS_COLS; ++c) o[c] = 0.0f;
        float den = 1.0f;
        if (MODE == 0) {
#pragma unroll
            for (int k = 0; k < NK; ++k) {
                const float a = expf(ls_logsigmoid(g[k] + bias[k]) * gate_param);      // gate_param = 1 / tau
#pragma unroll
                for (int c = 0; c < LS_COLS; ++c) {
                    S[k][c] = fmaf(a, S[k][c], kk[k] * v[c]);
                    o[c] = fmaf(S[k][c], q[k], o[c]);
                }
            }
        } else {
            const float cap = gate_param;
            const float li = cap * tanhf((gi + b_i) / cap);
            const float lf = ls_logsigmoid(cap * tanhf((gf + b_f) / cap));
            const float m_new = fmaxf(lf + m, li);
            const float keep = expf(lf + m - m_new), take = expf(li - m_new);
            m = m_new;
            float nq_dot = 0.0f;
#pragma unroll
            for (int k = 0; k < NK; ++k) {
                const float tk = take * kk[k];
                nvec[k] = fmaf(keep, nvec[k], tk);
                nq_dot = fmaf(nvec[k], q[k], nq_dot);
#pragma unroll
                for (int c = 0; c < LS_COLS; ++c) {
                    S[k][c] = fmaf(keep, S[k][c], tk * v[c]);
                    o[c] = fmaf(S[k][c], q[k], o[c]);
                }
            }
            nq_dot = ib_warp_sum(nq_dot);
            den = fmaxf(fabsf(nq_dot), expf(-m)) + 1e-6f;
        }
#pragma unroll
        for (int c = 0; c < LS_COLS; ++c) o[c] = ib_warp_sum(o[c]);
        if (lane < LS_COLS && e0 + lane < E) {
            float mine = o[0];
#pragma unroll
            for (int c = 1; c < LS_COLS; ++c) mine = lane == c ? o[c] : mine;
            out[((long)row * H + h) * E + e0 + lane] = MODE == 1 ? mine / den : mine;
        }
    }
#pragma unroll
    for (int k = 0; k < NK; ++k) {
        const int d = lane + 32 * k;
        if (d < D) {
#pragma unroll
            for (int c = 0; c < LS_COLS; ++c)
                if (e0 + c < E) st_S[(long)c * D + d] = S[k][c];
            if (MODE == 1 && e0 == 0) st_n[d] = nvec[k];
        }
    }
    if (MODE == 1 && e0 == 0 && lane == 0) *st_m = m;
}

// proj [rows, ld] act_t holds q and k as [H, D] and v as [H, E] from columns q_col, k_col, v_col on.
// gates [rows, ld_gates] float: mode 0 the decay's pre-activations [H, D] (gate_bias [H * D], gate_param = tau);
// mode 1 the input gate's and then the forget gate's pre-activations [2, H] (gate_bias [2 * H], gate_param = cap).
// out [rows, H, E] float.  state: see the head of the file; slot_stride floats per slot.
IB_EXPORT int ib_linear_scan(int mode, const void* proj, long ld, int q_col, int k_col, int v_col, const float* gates,
                             long ld_gates, const float* gate_bias, float gate_param, float q_scale, float* state,
                             long slot_stride, const int* q_start, const int* slots, int n_requests, float* out, int H,
                             int D, int E, cudaStream_t stream) {
    if (n_requests <= 0) return IB_OK;
    if (H <= 0 || D <= 0 || E <= 0 || proj == nullptr || gates == nullptr || gate_bias == nullptr || state == nullptr ||
        (mode != 0 && mode != 1) || !(gate_param > 0.0f))
        return IB_ERR_ARGUMENT;
    if (D > 256 || H > 65535 || n_requests > 65535) return IB_ERR_UNSUPPORTED;
    const long need = (long)H * E * D + (mode == 1 ? (long)H * D + H : 0);
    if (slot_stride < need) return IB_ERR_ARGUMENT;
    const dim3 grid((E + LS_WARPS * LS_COLS - 1) / (LS_WARPS * LS_COLS), H, n_requests);
    const float param = mode == 0 ? 1.0f / gate_param : gate_param;
#define IB_SCAN(MODE, NK)                                                                                          \
    ib_launch(linear_scan_kernel<MODE, NK>, grid, 32 * LS_WARPS, 0, stream, (const act_t*)proj, ld, q_col, k_col,  \
              v_col, gates, ld_gates, gate_bias, param, q_scale, state, slot_stride, q_start, slots, out, H, D, E)
#define IB_SCAN_NK(MODE)                                                                                           \
    do {                                                                                                           \
        if (D <= 32) IB_SCAN(MODE, 1); else if (D <= 64) IB_SCAN(MODE, 2);                                         \
        else if (D <= 128) IB_SCAN(MODE, 4); else IB_SCAN(MODE, 8);                                                \
    } while (0)
    if (mode == 0) IB_SCAN_NK(0); else IB_SCAN_NK(1);
#undef IB_SCAN_NK
#undef IB_SCAN
    return ib_launch_status();
}
