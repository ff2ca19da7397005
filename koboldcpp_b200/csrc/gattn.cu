// gattn.cu -- grouped-query softmax attention with a per-head sink over f32 key / value caches, and linear attention with a
// decayed state (include/b200_ggml_ops.h: b200_op_qkv_store, b200_op_sink_attn, b200_op_linear_attn_scan).
//
// Cache rows are indexed by cell, one row per token holding all kv heads; which cells a token sees follows from the (sequence,
// position) pairs of token and cell, so a batch may mix sequences, cells may be scattered, and a sliding window with kept first
// positions needs no mask tensor.  The sink only enters the softmax denominator.
#include "ops_util.cuh"
#include <cuda_bf16.h>

namespace b200 {
using namespace opx;

// ------------------------------------------------------------------------------------------------ bias + norm + rotation + cache store
// One CTA per token.  The RMS statistics run over the whole projection (all heads at once); q is rewritten in place, k and v go
// to the token's cache rows.
__global__ void __launch_bounds__(256) qkv_store_kernel(const b200_qkv_store_args a) {
    __shared__ float sh[32];
    const int t = blockIdx.x;
    const int nq = a.n_head * a.dim, nk = a.n_head_kv * a.dim, nv = a.n_head_kv * a.vdim;
    float *q = a.q + (int64_t)t * a.q_stride;
    const float *k = a.k + (int64_t)t * a.k_stride, *v = a.v + (int64_t)t * a.v_stride;
    const int64_t cell = a.cells[t];
    float *kc = a.k_cache + cell * a.k_cache_stride, *vc = a.v_cache + cell * a.v_cache_stride;
    float qs = 1.f, ks = 1.f;
    if (a.q_norm) {
        float s = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float x = q[i] + (a.q_bias ? a.q_bias[i] : 0.f); s += x * x; }
        qs = 1.0f / sqrtf(block_sum(s, sh) / (float)nq + a.eps);
    }
    if (a.k_norm) {
        float s = 0.f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float x = k[i] + (a.k_bias ? a.k_bias[i] : 0.f); s += x * x; }
        ks = 1.0f / sqrtf(block_sum(s, sh) / (float)nk + a.eps);
    }
    const float p = (float)a.pos[t];
    const int half = a.n_dims / 2, per_head = half + (a.dim - a.n_dims);  // work items of a head: rotated pairs, then single values
    for (int which = 0; which < 2; which++) {
        const float *src = which ? k : q;
        float *dst = which ? kc : q;
        const float *bias = which ? a.k_bias : a.q_bias, *nw = which ? a.k_norm : a.q_norm;
        const float sc = which ? ks : qs;
        const int heads = which ? a.n_head_kv : a.n_head;
        for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
            const int hh = idx / per_head, j = idx - hh * per_head;
            if (j >= half) {
                const int e = hh * a.dim + a.n_dims + (j - half);
                float x = src[e] + (bias ? bias[e] : 0.f);
                if (nw) x = x * sc * nw[e];
                dst[e] = x;
                continue;
            }
            const int e0 = hh * a.dim + 2 * j, e1 = e0 + 1;
            float u = src[e0] + (bias ? bias[e0] : 0.f), w = src[e1] + (bias ? bias[e1] : 0.f);
            if (nw) { u = u * sc * nw[e0]; w = w * sc * nw[e1]; }
            float sn, cs;
            sincosf(p * a.freqs[j], &sn, &cs);
            dst[e0] = u * cs - w * sn;
            dst[e1] = w * cs + u * sn;
        }
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) vc[i] = v[i] + (a.v_bias ? a.v_bias[i] : 0.f);
}

__device__ __forceinline__ bool sa_visible(int cell_seq, int cell_pos, int seq, int pos, int window, int keep_first) {
    return cell_seq == seq && cell_pos <= pos && (window <= 0 || pos - cell_pos < window || cell_pos < keep_first);
}

// ------------------------------------------------------------------------------------------------ attention, f32 products
// One CTA per (token, head); its warps stride over the cells 32 at a time (one visibility test per lane, one ballot), then work
// through the visible ones SA_UNROLL at a time with all loads of a round issued before the first dot product.  Each warp keeps an
// online softmax and an accumulator; they meet in shared memory, where the sink joins the denominator.
// ND = ceil(dim / 32), NV = ceil(vdim / 32): values per lane.  WARPS is 16 when there are few (token, head) pairs (decode).
constexpr int SA_UNROLL = 4;
template <int ND, int NV, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) sink_attn_kernel(const b200_sink_attn_args a) {
    extern __shared__ float smem[];  // [WARPS][vdim] accumulators, then m[WARPS], l[WARPS]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = a.dim, V = a.vdim;
    const int g = h / (a.n_head / a.n_head_kv);
    const float *qp = a.q + (int64_t)t * a.q_stride + (int64_t)h * D;
    const float *kb = a.k_cache + (int64_t)g * D, *vb = a.v_cache + (int64_t)g * V;
    float q[ND], acc[NV];
#pragma unroll
    for (int i = 0; i < ND; i++) { const int j = lane + 32 * i; q[i] = j < D ? qp[j] * a.scale : 0.f; }
#pragma unroll
    for (int i = 0; i < NV; i++) acc[i] = 0.f;
    const int seq = a.tok_seq[t], pos = a.tok_pos[t];
    float m = -INFINITY, l = 0.f;
    for (int cb = warp * 32; cb < a.n_kv; cb += WARPS * 32) {
        bool mine = false;
        if (cb + lane < a.n_kv) mine = sa_visible(a.cell_seq[cb + lane], a.cell_pos[cb + lane], seq, pos, a.window, a.keep_first);
        unsigned rest = __ballot_sync(0xffffffffu, mine);
        while (rest) {
            bool vis[SA_UNROLL];  // warp-uniform
            int cu[SA_UNROLL];
            float kv[SA_UNROLL][ND], vv[SA_UNROLL][NV];
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                vis[u] = rest != 0u;
                cu[u] = vis[u] ? cb + __ffs(rest) - 1 : 0;
                rest &= rest - 1;  // 0 stays 0
            }
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                if (!vis[u]) continue;
                const float *kr = kb + (int64_t)cu[u] * a.k_cache_stride, *vr = vb + (int64_t)cu[u] * a.v_cache_stride;
#pragma unroll
                for (int i = 0; i < ND; i++) { const int j = lane + 32 * i; kv[u][i] = j < D ? kr[j] : 0.f; }
#pragma unroll
                for (int i = 0; i < NV; i++) { const int j = lane + 32 * i; vv[u][i] = j < V ? vr[j] : 0.f; }
            }
            float s[SA_UNROLL];
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                s[u] = 0.f;
                if (!vis[u]) continue;
#pragma unroll
                for (int i = 0; i < ND; i++) s[u] += q[i] * kv[u][i];
            }
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) if (vis[u]) s[u] = warp_sum(s[u]);
#pragma unroll
            for (int u = 0; u < SA_UNROLL; u++) {
                if (!vis[u]) continue;
                const float mn = fmaxf(m, s[u]);
                const float corr = expf(m - mn), p = expf(s[u] - mn);  // m = -inf at the first cell: corr = 0
                l = l * corr + p;
#pragma unroll
                for (int i = 0; i < NV; i++) acc[i] = acc[i] * corr + p * vv[u][i];
                m = mn;
            }
        }
    }
    float *sacc = smem + (size_t)warp * V, *sm = smem + (size_t)WARPS * V, *sl = sm + WARPS;
#pragma unroll
    for (int i = 0; i < NV; i++) { const int j = lane + 32 * i; if (j < V) sacc[j] = acc[i]; }
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
    __syncthreads();
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    float M = sink;
    for (int w = 0; w < WARPS; w++) M = fmaxf(M, sm[w]);
    float L = a.sink ? expf(sink - M) : 0.f;
    for (int w = 0; w < WARPS; w++) if (sm[w] != -INFINITY) L += sl[w] * expf(sm[w] - M);
    __syncthreads();
    if (threadIdx.x < WARPS) sl[threadIdx.x] = sm[threadIdx.x] == -INFINITY ? 0.f : expf(sm[threadIdx.x] - M);  // the warp's weight in the merge
    __syncthreads();
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    float *out = a.dst + (int64_t)t * a.dst_stride + (int64_t)h * V;
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; w++) o += smem[(size_t)w * V + j] * sl[w];
        out[j] = o * inv;
    }
}

template <int ND, int NV, int WARPS>
static int launch_sink_attn3(const b200_sink_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)a->n_tokens, (unsigned)a->n_head);
    const size_t smem = ((size_t)WARPS * a->vdim + 2 * WARPS) * 4;
    sink_attn_kernel<ND, NV, WARPS><<<grid, WARPS * 32, smem, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
template <int ND, int NV>
static int launch_sink_attn2(const b200_sink_attn_args *a, cudaStream_t st) {
    if ((int64_t)a->n_tokens * a->n_head < 2 * 148 && a->n_kv > 64) return launch_sink_attn3<ND, NV, 16>(a, st);
    return launch_sink_attn3<ND, NV, 4>(a, st);
}
template <int ND>
static int launch_sink_attn(const b200_sink_attn_args *a, cudaStream_t st) {
    const int nv = (a->vdim + 31) / 32;
    if (nv <= 1) return launch_sink_attn2<ND, 1>(a, st);
    if (nv <= 2) return launch_sink_attn2<ND, 2>(a, st);
    if (nv <= 4) return launch_sink_attn2<ND, 4>(a, st);
    return launch_sink_attn2<ND, 8>(a, st);
}

// ------------------------------------------------------------------------------------------------ linear attention with decay
// The columns of the state never interact: a warp owns LA_CW columns of one (sequence, head) and keeps them in registers over
// the whole token loop, a lane the rows d = lane, lane + 32, ...  The inputs of LA_CHUNK tokens are staged in shared memory
// (activation applied once) while the serial loop only does the decayed rank-one update and the column sums.
constexpr int LA_CW = 4, LA_WARPS = 4, LA_COLS = LA_CW * LA_WARPS, LA_CHUNK = 16;
__device__ __forceinline__ float la_act(float x, int act) { return act ? x / (1.0f + expf(-x)) : x; }
template <int DPL>
__global__ void __launch_bounds__(LA_WARPS * 32) linear_attn_scan_kernel(const b200_linear_attn_args a) {
    extern __shared__ float sm_[];  // q [LA_CHUNK][dim], k [LA_CHUNK][dim], v [LA_CHUNK][LA_COLS]
    const int h = blockIdx.y, s = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int D = a.dim, V = a.vdim;
    const int first = a.seq_info[s], count = a.seq_info[a.n_seq + s], slot = a.seq_info[2 * a.n_seq + s], fresh = a.seq_info[3 * a.n_seq + s];
    if (count <= 0) return;
    const int cb = blockIdx.x * LA_COLS, col0 = cb + warp * LA_CW;
    float *sq = sm_, *sk = sq + LA_CHUNK * D, *sv = sk + LA_CHUNK * D;
    float *Sp = a.state + (int64_t)slot * a.slot_stride + ((int64_t)h * V + col0) * D;
    const float decay = a.decay[h];
    float S[LA_CW][DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < LA_CW; c++) S[c][i] = (!fresh && d < D && col0 + c < V) ? Sp[(int64_t)c * D + d] : 0.f;
    }
    for (int t0 = 0; t0 < count; t0 += LA_CHUNK) {
        const int nt = min(LA_CHUNK, count - t0);
        __syncthreads();  // the previous chunk has been read
        for (int idx = tid; idx < nt * D; idx += LA_WARPS * 32) {
            const int tt = idx / D, d = idx - tt * D;
            const int64_t tok = first + t0 + tt;
            sq[idx] = la_act(a.q[tok * a.q_stride + (int64_t)h * D + d], a.act);
            sk[idx] = la_act(a.k[tok * a.k_stride + (int64_t)h * D + d], a.act);
        }
        for (int idx = tid; idx < nt * LA_COLS; idx += LA_WARPS * 32) {
            const int tt = idx / LA_COLS, c = idx - tt * LA_COLS;
            const int64_t tok = first + t0 + tt;
            sv[idx] = cb + c < V ? la_act(a.v[tok * a.v_stride + (int64_t)h * V + cb + c], a.act) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            float qv[DPL], kv[DPL], part[LA_CW];
#pragma unroll
            for (int i = 0; i < DPL; i++) { const int d = lane + 32 * i; qv[i] = d < D ? sq[tt * D + d] : 0.f; kv[i] = d < D ? sk[tt * D + d] : 0.f; }
#pragma unroll
            for (int c = 0; c < LA_CW; c++) {
                const float vc = sv[tt * LA_COLS + warp * LA_CW + c];
                part[c] = 0.f;
#pragma unroll
                for (int i = 0; i < DPL; i++) { S[c][i] = decay * S[c][i] + kv[i] * vc; part[c] += S[c][i] * qv[i]; }
            }
#pragma unroll
            for (int c = 0; c < LA_CW; c++) part[c] = warp_sum(part[c]);
            if (lane < LA_CW && col0 + lane < V) {
                float o = part[0];
#pragma unroll
                for (int c = 1; c < LA_CW; c++) if (lane == c) o = part[c];
                a.dst[(int64_t)(first + t0 + tt) * a.dst_stride + (int64_t)h * V + col0 + lane] = o;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < LA_CW; c++) if (d < D && col0 + c < V) Sp[(int64_t)c * D + d] = S[c][i];
    }
}

template <int DPL>
static int launch_linear_attn(const b200_linear_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)((a->vdim + LA_COLS - 1) / LA_COLS), (unsigned)a->heads, (unsigned)a->n_seq);
    const size_t smem = (size_t)LA_CHUNK * (2 * a->dim + LA_COLS) * 4;
    linear_attn_scan_kernel<DPL><<<grid, LA_WARPS * 32, smem, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_op_qkv_store(const b200_qkv_store_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k && a->v && a->pos && a->cells && a->k_cache && a->v_cache && (a->freqs || a->n_dims == 0), B200_ERR_INVALID, "b200_op_qkv_store: NULL argument");
    OPX_REQUIRE(a->n_head > 0 && a->n_head_kv > 0 && a->n_head % a->n_head_kv == 0 && a->dim > 0 && a->vdim > 0 && a->n_dims >= 0 && a->n_dims % 2 == 0 && a->n_dims <= a->dim &&
                a->n_tokens >= 0 && a->k_cache_stride >= (int64_t)a->n_head_kv * a->dim && a->v_cache_stride >= (int64_t)a->n_head_kv * a->vdim, B200_ERR_INVALID,
                "b200_op_qkv_store: bad sizes");
    if (a->n_tokens == 0) return B200_OK;
    qkv_store_kernel<<<(unsigned)a->n_tokens, 256, 0, (cudaStream_t)stream>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_sink_attn(const b200_sink_attn_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k_cache && a->v_cache && a->cell_seq && a->cell_pos && a->tok_seq && a->tok_pos && a->dst, B200_ERR_INVALID, "b200_op_sink_attn: NULL argument");
    OPX_REQUIRE(a->n_head > 0 && a->n_head <= 65535 && a->n_head_kv > 0 && a->n_head % a->n_head_kv == 0 && a->dim > 0 && a->dim <= 256 && a->vdim > 0 && a->vdim <= 256 &&
                a->n_tokens >= 0 && a->n_kv >= 0 && a->window >= 0 && a->keep_first >= 0, B200_ERR_UNSUPPORTED, "b200_op_sink_attn: head sizes up to 256, heads up to 65535");
    if (a->n_tokens == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    const int nd = (a->dim + 31) / 32;
    if (nd <= 1) return launch_sink_attn<1>(a, st);
    if (nd <= 2) return launch_sink_attn<2>(a, st);
    if (nd <= 4) return launch_sink_attn<4>(a, st);
    return launch_sink_attn<8>(a, st);
}

extern "C" int b200_op_linear_attn_scan(const b200_linear_attn_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q && a->k && a->v && a->decay && a->seq_info && a->state && a->dst, B200_ERR_INVALID, "b200_op_linear_attn_scan: NULL argument");
    OPX_REQUIRE(a->heads > 0 && a->heads <= 65535 && a->dim > 0 && a->dim <= 256 && a->vdim > 0 && a->n_seq >= 0 && a->n_seq <= 65535 &&
                a->slot_stride >= (int64_t)a->heads * a->dim * a->vdim, B200_ERR_UNSUPPORTED, "b200_op_linear_attn_scan: dim up to 256");
    if (a->n_seq == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    const int dpl = (a->dim + 31) / 32;
    if (dpl <= 1) return launch_linear_attn<1>(a, st);
    if (dpl <= 2) return launch_linear_attn<2>(a, st);
    if (dpl <= 4) return launch_linear_attn<4>(a, st);
    return launch_linear_attn<8>(a, st);
}
