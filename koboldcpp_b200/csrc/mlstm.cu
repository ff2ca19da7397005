// mlstm.cu -- matrix-memory recurrence (mLSTM) with a stabilised exponential input gate (include/b200_ggml_ops.h: b200_op_mlstm_scan).
//
// Per (sequence, head) the state is a dim x vdim matrix S, a dim vector n and a running maximum m, all f32 and carried from
// token to token in a slot of the state pool.  The columns of S never interact: a CTA owns 16 or 32 columns of one (sequence, head),
// a warp 2 or 4 of them, a lane the rows d = lane, lane + 32, ... -- the state stays in registers for the whole token loop, the
// per-token inputs come through shared memory a chunk of tokens at a time.  The sums over the rows (n . q and one numerator per
// column) do not feed the recurrence, so the token loop only parks each lane's share in shared memory and the warp adds them
// up for ML_RG tokens at a time, one sum per lane, outside the serial chain.
// n . q and m are recomputed by every warp (dim MACs) instead of being exchanged.
#include "ops_util.cuh"

namespace b200 {
using namespace opx;

constexpr int ML_WARPS = 8, ML_CHUNK = 16, ML_THREADS = ML_WARPS * 32;
constexpr int ML_RG = 8;  // tokens whose reductions are done together
// A warp owns CW columns (2 or 4: a CTA 16 or 32).  4 does less of the work that every warp repeats (n, n . q); 2 gives twice the
// CTAs when heads x columns / 32 would leave SMs idle.  n and m belong to the head, not to a column: the state keeps one copy
// per ML_LAYOUT_COLS columns so that no CTA reads what another CTA of the same launch writes, every copy is the same, and a
// CTA of 32 columns reads the first of its two copies and writes both -- launches with either CW can follow each other.
constexpr int ML_LAYOUT_COLS = 16;

// The inputs of ML_CHUNK tokens (q, k of the head, v of the CTA's columns, the two gate values) are fetched by all threads
// at once into registers while the previous chunk is being processed, then parked in shared memory, with the gate
// non-linearities (tanh cap, log-sigmoid) already applied by one thread per token: the serial token loop reads shared memory
// only and pays two exponentials per token, and a chunk costs one round trip to L2 that overlaps the chunk before it.
template <int DPL, int ML_CW>
__global__ void __launch_bounds__(ML_THREADS) mlstm_scan_kernel(const b200_mlstm_args a) {
    extern __shared__ float sm_[];
    constexpr int ML_COLS = ML_CW * ML_WARPS, ML_NP = ML_CW + 1, ML_COPIES = ML_COLS / ML_LAYOUT_COLS;  // ML_NP: sums per token (n . q and one numerator per column)
    const int h = blockIdx.y, s = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int H = a.heads, D = a.dim, V = a.vdim;
    const int first = a.seq_info[s], count = a.seq_info[a.n_seq + s], slot = a.seq_info[2 * a.n_seq + s], fresh = a.seq_info[3 * a.n_seq + s];
    const int cb = blockIdx.x * ML_COLS, col0 = cb + warp * ML_CW;
    const bool active = col0 < V && count > 0;
    float *sq = sm_, *sk = sq + ML_CHUNK * D, *sv = sk + ML_CHUNK * D, *sli = sv + ML_CHUNK * ML_COLS, *slf = sli + ML_CHUNK;
    float *wpart = slf + ML_CHUNK + warp * (ML_RG * ML_NP * 32 + ML_RG * ML_NP + ML_RG), *wred = wpart + ML_RG * ML_NP * 32, *wmn = wred + ML_RG * ML_NP;  // this warp's own
    float S[ML_CW][DPL], nn[DPL], m = 0.f;
    // n and m are kept once per CTA (column tile): a CTA never reads state that another CTA of the same launch writes
    const int nvt = (V + ML_LAYOUT_COLS - 1) / ML_LAYOUT_COLS, vt0 = blockIdx.x * ML_COPIES;
    float *base = a.state + (int64_t)slot * a.slot_stride;
    float *Sp = base + ((int64_t)h * V + col0) * D;
    float *np = base + (int64_t)H * V * D + ((int64_t)h * nvt + vt0) * D;
    float *mp = base + (int64_t)H * V * D + (int64_t)H * nvt * D + (int64_t)h * nvt + vt0;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
        const bool ok = active && d < D && !fresh;
        nn[i] = ok ? np[d] : 0.f;
#pragma unroll
        for (int c = 0; c < ML_CW; c++) S[c][i] = ok && col0 + c < V ? Sp[(int64_t)c * D + d] : 0.f;
    }
    if (active && !fresh) m = *mp;
    const float cap = a.gate_cap, inv_cap = 1.0f / a.gate_cap, ib = a.i_bias ? a.i_bias[h] : 0.f, fb = a.f_bias ? a.f_bias[h] : 0.f;
    // per thread and chunk: NQK values of q and of k, 2 of v, one token's gates (threads < ML_CHUNK)
    constexpr int NQK = (ML_CHUNK * 32 * DPL + ML_THREADS - 1) / ML_THREADS, NV = ML_CHUNK * ML_COLS / ML_THREADS;
    float pq[NQK], pk[NQK], pv[NV], pgi = 0.f, pgf = 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(ML_CHUNK, count - t0);
#pragma unroll
        for (int j = 0; j < NQK; j++) {
            const int idx = tid + j * ML_THREADS, tk = idx / D, d = idx - tk * D;
            const bool ok = tk < nt;
            const int64_t tok = first + t0 + tk;
            pq[j] = ok ? a.q[tok * a.q_stride + (int64_t)h * D + d] * a.q_scale : 0.f;
            pk[j] = ok ? a.k[tok * a.k_stride + (int64_t)h * D + d] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const int idx = tid + j * ML_THREADS, tk = idx / ML_COLS, c = idx - tk * ML_COLS;
            pv[j] = (tk < nt && cb + c < V) ? a.v[(int64_t)(first + t0 + tk) * a.v_stride + (int64_t)h * V + cb + c] : 0.f;
        }
        if (tid < nt) { pgi = a.ig[(int64_t)(first + t0 + tid) * a.g_stride + h]; pgf = a.fg[(int64_t)(first + t0 + tid) * a.g_stride + h]; }
    };
    auto park = [&]() {
#pragma unroll
        for (int j = 0; j < NQK; j++) { const int idx = tid + j * ML_THREADS; if (idx < ML_CHUNK * D) { sq[idx] = pq[j]; sk[idx] = pk[j]; } }
#pragma unroll
        for (int j = 0; j < NV; j++) sv[tid + j * ML_THREADS] = pv[j];
        if (tid < ML_CHUNK) {
            sli[tid] = cap * tanhf((pgi + ib) * inv_cap);
            const float x = cap * tanhf((pgf + fb) * inv_cap);
            slf[tid] = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));  // log sigmoid(x)
        }
    };
    if (count > 0) fetch(0);
    for (int t0 = 0; t0 < count; t0 += ML_CHUNK) {
        __syncthreads();  // the previous chunk has been read
        park();
        __syncthreads();
        if (t0 + ML_CHUNK < count) fetch(t0 + ML_CHUNK);  // in flight while this chunk is processed
        if (!active) continue;
        const int nt = min(ML_CHUNK, count - t0);
        for (int g0 = 0; g0 < nt; g0 += ML_RG) {
            const int ng = min(ML_RG, nt - g0);
            for (int tg = 0; tg < ng; tg++) {
                const int t = g0 + tg;
                const float li = sli[t], lf = slf[t];
                const float mn = fmaxf(lf + m, li);
                const float fa = expf(lf + m - mn), fi = expf(li - mn);
                float cv[ML_CW], dn = 0.f, num[ML_CW];
#pragma unroll
                for (int c = 0; c < ML_CW; c++) { cv[c] = sv[t * ML_COLS + warp * ML_CW + c]; num[c] = 0.f; }
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    const int d = lane + 32 * i;
                    const float cq = d < D ? sq[t * D + d] : 0.f, bk = d < D ? fi * sk[t * D + d] : 0.f;
                    nn[i] = fa * nn[i] + bk;
                    dn += nn[i] * cq;
#pragma unroll
                    for (int c = 0; c < ML_CW; c++) {
                        S[c][i] = fa * S[c][i] + bk * cv[c];
                        num[c] += S[c][i] * cq;
                    }
                }
                // the lane's shares of n . q and of the ML_CW numerators wait in shared memory: nothing of the recurrence depends on them
                float *pp = wpart + tg * ML_NP * 32;
                pp[lane] = dn;
#pragma unroll
                for (int c = 0; c < ML_CW; c++) pp[(1 + c) * 32 + lane] = num[c];
                if (lane == 0) wmn[tg] = mn;
                m = mn;
            }
            __syncwarp();
            // ng * ML_NP sums of 32 shares each, one sum per lane; lane L starts at share L so that the lanes hit different banks
            for (int p = lane; p < ng * ML_NP; p += 32) {
                const float *pp = wpart + p * 32;
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int i = 0; i < 32; i += 2) { s0 += pp[(i + lane) & 31]; s1 += pp[(i + 1 + lane) & 31]; }
                wred[p] = s0 + s1;
            }
            __syncwarp();
            for (int idx = lane; idx < ng * ML_CW; idx += 32) {
                const int tg = idx / ML_CW, c = idx - tg * ML_CW;
                const float den = fmaxf(fabsf(wred[tg * ML_NP]), expf(-wmn[tg])) + 1e-6f;
                if (col0 + c < V) a.dst[(int64_t)(first + t0 + g0 + tg) * a.dst_stride + (int64_t)h * V + col0 + c] = wred[tg * ML_NP + 1 + c] / den;
            }
            __syncwarp();
        }
    }
    if (!active) return;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
        if (d >= D) continue;
        if (warp < ML_COPIES && vt0 + warp < nvt) np[(int64_t)warp * D + d] = nn[i];
#pragma unroll
        for (int c = 0; c < ML_CW; c++) if (col0 + c < V) Sp[(int64_t)c * D + d] = S[c][i];
    }
    if (warp < ML_COPIES && vt0 + warp < nvt && lane == 0) mp[warp] = m;
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_mlstm_state_floats(int32_t heads, int32_t dim, int32_t vdim) {
    const int64_t nvt = (vdim + ML_LAYOUT_COLS - 1) / ML_LAYOUT_COLS;
    return (int64_t)heads * vdim * dim + (int64_t)heads * nvt * dim + (int64_t)heads * nvt;
}

extern "C" int b200_op_mlstm_scan(const b200_mlstm_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k && a->v && a->ig && a->fg && a->seq_info && a->state && a->dst, B200_ERR_INVALID, "b200_op_mlstm_scan: NULL argument");
    OPX_REQUIRE(a->heads > 0 && a->heads <= 65535 && a->dim > 0 && a->dim <= 512 && a->vdim > 0 && a->n_seq >= 0 && a->n_seq <= 65535 && a->gate_cap > 0.f &&
                a->slot_stride >= b200_mlstm_state_floats(a->heads, a->dim, a->vdim), B200_ERR_UNSUPPORTED,
                "b200_op_mlstm_scan: dim <= 512, heads and sequences <= 65535, gate_cap > 0");
    if (a->n_seq == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    const int dpl = (a->dim + 31) / 32;
    // 4 columns per warp when that still gives every SM a CTA, else 2
    const bool wide = (int64_t)((a->vdim + 31) / 32) * a->heads * a->n_seq >= 120;
    const int cols = (wide ? 4 : 2) * ML_WARPS, np_ = (wide ? 4 : 2) + 1;
    const dim3 grid((unsigned)((a->vdim + cols - 1) / cols), (unsigned)a->heads, (unsigned)a->n_seq);
    const size_t smem = ((size_t)2 * ML_CHUNK * a->dim + ML_CHUNK * cols + 2 * ML_CHUNK + (size_t)ML_WARPS * (ML_RG * np_ * 32 + ML_RG * np_ + ML_RG)) * 4;
#define B200_ML_LAUNCH2(N, C)                                                                                                                    \
    do {                                                                                                                                         \
        if (smem > 48 * 1024) B200_CUDA_TRY(cudaFuncSetAttribute(mlstm_scan_kernel<N, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        mlstm_scan_kernel<N, C><<<grid, ML_THREADS, smem, st>>>(*a);                                                                             \
    } while (0)
#define B200_ML_LAUNCH(N)               \
    do {                                \
        if (wide) B200_ML_LAUNCH2(N, 4); \
        else B200_ML_LAUNCH2(N, 2);     \
    } while (0)
    if (dpl <= 1) B200_ML_LAUNCH(1);
    else if (dpl <= 2) B200_ML_LAUNCH(2);
    else if (dpl <= 4) B200_ML_LAUNCH(4);
    else if (dpl <= 8) B200_ML_LAUNCH(8);
    else B200_ML_LAUNCH(16);
#undef B200_ML_LAUNCH2
#undef B200_ML_LAUNCH
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
