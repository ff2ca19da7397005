// mlstm.cu -- matrix-memory recurrence (mLSTM) with a stabilised exponential input gate (include/b200_ggml_ops.h: b200_op_mlstm_scan).
//
// Per (sequence, head) the state is a dim x vdim matrix S, a dim vector n and a running maximum m, all f32 and carried from
// token to token in a slot of the state pool.  The columns of S never interact: a CTA owns 32 columns of one (sequence, head),
// a warp 4 of them, a lane the rows d = lane, lane + 32, ... -- the state stays in registers for the whole token loop, the
// per-token inputs (q, k, v, two gate values) are prefetched one token ahead, and a token costs one warp reduction per column.
// n . q and m are recomputed by every warp (dim MACs) instead of being exchanged.
#include "ops_util.cuh"

namespace b200 {
using namespace opx;

constexpr int ML_CW = 4, ML_WARPS = 8, ML_COLS = ML_CW * ML_WARPS;

template <int DPL>
__global__ void __launch_bounds__(ML_WARPS * 32) mlstm_scan_kernel(const b200_mlstm_args a) {
    const int h = blockIdx.y, s = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = a.heads, D = a.dim, V = a.vdim;
    const int first = a.seq_info[s], count = a.seq_info[a.n_seq + s], slot = a.seq_info[2 * a.n_seq + s], fresh = a.seq_info[3 * a.n_seq + s];
    const int col0 = blockIdx.x * ML_COLS + warp * ML_CW;
    const bool active = col0 < V && count > 0;
    float S[ML_CW][DPL], nn[DPL], m = 0.f;
    // n and m are kept once per CTA (column tile): a CTA never reads state that another CTA of the same launch writes
    const int nvt = gridDim.x;
    float *base = a.state + (int64_t)slot * a.slot_stride;
    float *Sp = base + ((int64_t)h * V + col0) * D;
    float *np = base + (int64_t)H * V * D + ((int64_t)h * nvt + blockIdx.x) * D;
    float *mp = base + (int64_t)H * V * D + (int64_t)H * nvt * D + (int64_t)h * nvt + blockIdx.x;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
        const bool ok = active && d < D && !fresh;
        nn[i] = ok ? np[d] : 0.f;
#pragma unroll
        for (int c = 0; c < ML_CW; c++) S[c][i] = ok && col0 + c < V ? Sp[(int64_t)c * D + d] : 0.f;
    }
    if (active && !fresh) m = *mp;
    __syncthreads();  // warp 0 rewrites n and m at the end: every warp has read them by now
    if (!active) return;
    const float cap = a.gate_cap, inv_cap = 1.0f / a.gate_cap, ib = a.i_bias ? a.i_bias[h] : 0.f, fb = a.f_bias ? a.f_bias[h] : 0.f;
    float q[DPL], k[DPL], v[ML_CW], gi, gf;
    auto load = [&](int tok) {
        const float *qp = a.q + (int64_t)tok * a.q_stride + (int64_t)h * D, *kp = a.k + (int64_t)tok * a.k_stride + (int64_t)h * D;
        const float *vp = a.v + (int64_t)tok * a.v_stride + (int64_t)h * V + col0;
#pragma unroll
        for (int i = 0; i < DPL; i++) { const int d = lane + 32 * i; q[i] = d < D ? qp[d] * a.q_scale : 0.f; k[i] = d < D ? kp[d] : 0.f; }
#pragma unroll
        for (int c = 0; c < ML_CW; c++) v[c] = col0 + c < V ? vp[c] : 0.f;
        gi = a.ig[(int64_t)tok * a.g_stride + h];
        gf = a.fg[(int64_t)tok * a.g_stride + h];
    };
    load(first);
    for (int t = 0; t < count; t++) {
        const int tok = first + t;
        float cq[DPL], ck[DPL], cv[ML_CW];
        const float ci = gi, cf = gf;
#pragma unroll
        for (int i = 0; i < DPL; i++) { cq[i] = q[i]; ck[i] = k[i]; }
#pragma unroll
        for (int c = 0; c < ML_CW; c++) cv[c] = v[c];
        if (t + 1 < count) load(tok + 1);
        const float li = cap * tanhf((ci + ib) * inv_cap);
        const float x = cap * tanhf((cf + fb) * inv_cap);
        const float lf = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));  // log sigmoid(x)
        const float mn = fmaxf(lf + m, li);
        const float fa = expf(lf + m - mn), fi = expf(li - mn);
        float dn = 0.f, num[ML_CW];
#pragma unroll
        for (int c = 0; c < ML_CW; c++) num[c] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            const float bk = fi * ck[i];
            nn[i] = fa * nn[i] + bk;
            dn += nn[i] * cq[i];
#pragma unroll
            for (int c = 0; c < ML_CW; c++) {
                S[c][i] = fa * S[c][i] + bk * cv[c];
                num[c] += S[c][i] * cq[i];
            }
        }
        dn = warp_sum(dn);
#pragma unroll
        for (int c = 0; c < ML_CW; c++) num[c] = warp_sum(num[c]);
        const float den = fmaxf(fabsf(dn), expf(-mn)) + 1e-6f;
        m = mn;
        float o = num[0];
#pragma unroll
        for (int c = 1; c < ML_CW; c++) if (lane == c) o = num[c];
        if (lane < ML_CW && col0 + lane < V) a.dst[(int64_t)tok * a.dst_stride + (int64_t)h * V + col0 + lane] = o / den;
    }
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
        if (d >= D) continue;
        if (warp == 0) np[d] = nn[i];
#pragma unroll
        for (int c = 0; c < ML_CW; c++) if (col0 + c < V) Sp[(int64_t)c * D + d] = S[c][i];
    }
    if (warp == 0 && lane == 0) *mp = m;
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_mlstm_state_floats(int32_t heads, int32_t dim, int32_t vdim) {
    const int64_t nvt = (vdim + ML_COLS - 1) / ML_COLS;
    return (int64_t)heads * vdim * dim + (int64_t)heads * nvt * dim + (int64_t)heads * nvt;
}

extern "C" int b200_op_mlstm_scan(const b200_mlstm_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k && a->v && a->ig && a->fg && a->seq_info && a->state && a->dst, B200_ERR_INVALID, "b200_op_mlstm_scan: NULL argument");
    OPX_REQUIRE(a->heads > 0 && a->heads <= 65535 && a->dim > 0 && a->dim <= 512 && a->vdim > 0 && a->n_seq >= 0 && a->n_seq <= 65535 && a->gate_cap > 0.f &&
                a->slot_stride >= b200_mlstm_state_floats(a->heads, a->dim, a->vdim), B200_ERR_UNSUPPORTED,
                "b200_op_mlstm_scan: dim <= 512, heads and sequences <= 65535, gate_cap > 0");
    if (a->n_seq == 0) return B200_OK;
    const dim3 grid((unsigned)((a->vdim + ML_COLS - 1) / ML_COLS), (unsigned)a->heads, (unsigned)a->n_seq);
    const cudaStream_t st = (cudaStream_t)stream;
    const int dpl = (a->dim + 31) / 32;
    if (dpl <= 1) mlstm_scan_kernel<1><<<grid, ML_WARPS * 32, 0, st>>>(*a);
    else if (dpl <= 2) mlstm_scan_kernel<2><<<grid, ML_WARPS * 32, 0, st>>>(*a);
    else if (dpl <= 4) mlstm_scan_kernel<4><<<grid, ML_WARPS * 32, 0, st>>>(*a);
    else if (dpl <= 8) mlstm_scan_kernel<8><<<grid, ML_WARPS * 32, 0, st>>>(*a);
    else mlstm_scan_kernel<16><<<grid, ML_WARPS * 32, 0, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
