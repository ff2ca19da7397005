// lattn.cu -- attention over a latent KV cache (include/b200_ggml_ops.h: b200_op_latent_kv_store, b200_op_latent_attn).
//
// A cache row holds kv_rank normalised latent values followed by rot_dim rotated key values; all heads read the same rows.
// With the key up-projection folded into the query (q_lat = W_uk^T q) and the value up-projection applied after the weighted
// sum, one head's work per cell is a dot product over the whole row and an axpy over its first kv_rank values, so the cache is
// streamed once per (token, head group) and never expanded to per-head keys and values in HBM.
// Visibility is decided per (token, cell) from (sequence, position) pairs: no mask tensor is built, uploaded or read.
#include "ops_util.cuh"

namespace b200 {
using namespace opx;

__global__ void latent_kv_store_kernel(const float *__restrict__ dkv, int64_t dkv_stride, const float *__restrict__ w, const int32_t *__restrict__ pos,
                                       const float *__restrict__ freqs, const int32_t *__restrict__ cells, float *__restrict__ cache, int64_t cache_stride,
                                       int kv_rank, int rot_dim, int n_dims, float mscale, float eps) {
    __shared__ float sh[32];
    const int t = blockIdx.x;
    const float *x = dkv + (int64_t)t * dkv_stride;
    float *row = cache + (int64_t)cells[t] * cache_stride;
    float s = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) s += x[i] * x[i];
    s = block_sum(s, sh);
    const float scale = 1.0f / sqrtf(s / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) row[i] = x[i] * scale * w[i];
    const float *xr = x + kv_rank;
    float *rr = row + kv_rank;
    const int half = n_dims / 2;
    const float p = (float)pos[t];
    for (int j = threadIdx.x; j < half + (rot_dim - n_dims); j += blockDim.x) {
        if (j >= half) { rr[n_dims + j - half] = xr[n_dims + j - half]; continue; }
        float sn, cs;
        sincosf(p * freqs[j], &sn, &cs);
        sn *= mscale; cs *= mscale;
        const float u = xr[2 * j], v = xr[2 * j + 1];
        rr[2 * j] = u * cs - v * sn;
        rr[2 * j + 1] = v * cs + u * sn;
    }
}

// One CTA per (token, head); its warps stride over the cells, each keeping an online softmax and a latent accumulator that are
// merged through shared memory at the end.  A warp takes LA_UNROLL cells per round: the visibility tests and the row loads of
// the whole round are issued before the first dot product, so a round pays the L2 latency once instead of once per cell.
// WARPS is 4 for prompt batches (many CTAs) and 16 when there are few (token, head) pairs (decode), where the cells of one
// pair are the only parallelism there is.  NL = ceil(kv_rank / 32), NR = ceil(rot_dim / 32): values per lane.
constexpr int LA_UNROLL = 4;
template <int NL, int NR, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) latent_attn_kernel(const b200_latent_attn_args a) {
    extern __shared__ float smem[];  // [WARPS][kv_rank] accumulators, then m[WARPS], l[WARPS]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KR = a.kv_rank, R = a.rot_dim;
    const float *ql = a.q_lat + (int64_t)h * a.q_lat_s_head + (int64_t)t * a.q_lat_s_tok;
    const float *qr = a.q_rot + (int64_t)h * a.q_rot_s_head + (int64_t)t * a.q_rot_s_tok;
    float q1[NL], q2[NR], acc[NL];
#pragma unroll
    for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; q1[i] = j < KR ? ql[j] * a.scale : 0.f; acc[i] = 0.f; }
#pragma unroll
    for (int i = 0; i < NR; i++) { const int j = lane + 32 * i; q2[i] = j < R ? qr[j] * a.scale : 0.f; }
    const int seq = a.tok_seq[t], pos = a.tok_pos[t];
    const int lo = a.window > 0 ? pos - a.window : INT_MIN;
    float m = -INFINITY, l = 0.f;
    for (int c0 = warp * LA_UNROLL; c0 < a.n_kv; c0 += WARPS * LA_UNROLL) {
        bool vis[LA_UNROLL];
        float rv[LA_UNROLL][NL], rr[LA_UNROLL][NR];
#pragma unroll
        for (int u = 0; u < LA_UNROLL; u++) {
            const int c = c0 + u;
            const int cp = c < a.n_kv ? a.cell_pos[c] : -1;
            vis[u] = c < a.n_kv && a.cell_seq[c] == seq && cp <= pos && cp > lo;  // warp-uniform
        }
#pragma unroll
        for (int u = 0; u < LA_UNROLL; u++) {
            if (!vis[u]) continue;
            const float *row = a.cache + (int64_t)(c0 + u) * a.cache_stride;
#pragma unroll
            for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; rv[u][i] = j < KR ? row[j] : 0.f; }
#pragma unroll
            for (int i = 0; i < NR; i++) { const int j = lane + 32 * i; rr[u][i] = j < R ? row[KR + j] : 0.f; }
        }
        float s[LA_UNROLL];
#pragma unroll
        for (int u = 0; u < LA_UNROLL; u++) {
            s[u] = 0.f;
            if (!vis[u]) continue;
#pragma unroll
            for (int i = 0; i < NL; i++) s[u] += q1[i] * rv[u][i];
#pragma unroll
            for (int i = 0; i < NR; i++) s[u] += q2[i] * rr[u][i];
        }
#pragma unroll
        for (int u = 0; u < LA_UNROLL; u++) if (vis[u]) s[u] = warp_sum(s[u]);
#pragma unroll
        for (int u = 0; u < LA_UNROLL; u++) {
            if (!vis[u]) continue;
            const float mn = fmaxf(m, s[u]);
            const float corr = expf(m - mn), p = expf(s[u] - mn);  // m = -inf at the first cell: corr = 0
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < NL; i++) acc[i] = acc[i] * corr + p * rv[u][i];
            m = mn;
        }
    }
    float *sacc = smem + (size_t)warp * KR, *sm = smem + (size_t)WARPS * KR, *sl = sm + WARPS;
#pragma unroll
    for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; if (j < KR) sacc[j] = acc[i]; }
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
    const float inv = 1.0f / L;
    float *out = a.dst + (int64_t)h * a.dst_s_head + (int64_t)t * a.dst_s_tok;
    for (int j = threadIdx.x; j < KR; j += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; w++) o += smem[(size_t)w * KR + j] * sl[w];
        out[j] = o * inv;
    }
}


// Prompt batches: one CTA per (token, group of 8 heads), one warp per head.  All heads of a token see the same cells, so the CTA
// stages a tile of LT_CELLS visible rows in shared memory once and every warp reads it from there: the cache rows cross L2 -> SM
// once per 8 (token, head) pairs instead of once per pair, which is what bounded the kernel above on prompts.  Tiles without a
// visible cell are skipped before anything is loaded.  Rows must be a multiple of 4 floats (16-byte copies).
constexpr int LT_HEADS = 8, LT_CELLS = 16;
template <int NL, int NR>
__global__ void __launch_bounds__(LT_HEADS * 32) latent_attn_tile_kernel(const b200_latent_attn_args a) {
    extern __shared__ float4 tile4[];  // [LT_CELLS][row floats]
    float *tile = reinterpret_cast<float *>(tile4);
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * LT_HEADS + warp;
    const bool head_ok = h < a.n_head;
    const int KR = a.kv_rank, R = a.rot_dim, RS = KR + R, RS4 = RS / 4;
    float q1[NL], q2[NR], acc[NL];
    {
        const float *ql = a.q_lat + (int64_t)(head_ok ? h : 0) * a.q_lat_s_head + (int64_t)t * a.q_lat_s_tok;
        const float *qr = a.q_rot + (int64_t)(head_ok ? h : 0) * a.q_rot_s_head + (int64_t)t * a.q_rot_s_tok;
#pragma unroll
        for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; q1[i] = j < KR ? ql[j] * a.scale : 0.f; acc[i] = 0.f; }
#pragma unroll
        for (int i = 0; i < NR; i++) { const int j = lane + 32 * i; q2[i] = j < R ? qr[j] * a.scale : 0.f; }
    }
    const int seq = a.tok_seq[t], pos = a.tok_pos[t];
    const int lo = a.window > 0 ? pos - a.window : INT_MIN;
    float m = -INFINITY, l = 0.f;
    for (int c0 = 0; c0 < a.n_kv; c0 += LT_CELLS) {
        bool vis = false;
        if (lane < LT_CELLS && c0 + lane < a.n_kv) {
            const int cp = a.cell_pos[c0 + lane];
            vis = a.cell_seq[c0 + lane] == seq && cp <= pos && cp > lo;
        }
        const unsigned mask = __ballot_sync(0xffffffffu, vis);  // the same in every warp
        if (!mask) continue;
        __syncthreads();  // the previous tile has been read
        for (int idx = threadIdx.x; idx < LT_CELLS * RS4; idx += LT_HEADS * 32) {
            const int u = idx / RS4, j = idx - u * RS4;
            if ((mask >> u) & 1u) tile4[idx] = reinterpret_cast<const float4 *>(a.cache + (int64_t)(c0 + u) * a.cache_stride)[j];
        }
        __syncthreads();
        for (unsigned rest = mask; rest; rest &= rest - 1) {
            const float *row = tile + (__ffs(rest) - 1) * RS;
            float rv[NL], s = 0.f;
#pragma unroll
            for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; rv[i] = j < KR ? row[j] : 0.f; s += q1[i] * rv[i]; }
#pragma unroll
            for (int i = 0; i < NR; i++) { const int j = lane + 32 * i; s += q2[i] * (j < R ? row[KR + j] : 0.f); }
            s = warp_sum(s);
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn), p = expf(s - mn);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < NL; i++) acc[i] = acc[i] * corr + p * rv[i];
            m = mn;
        }
    }
    if (!head_ok) return;
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    const float M = fmaxf(m, sink);
    const float f = m == -INFINITY ? 0.f : expf(m - M);
    const float inv = 1.0f / (l * f + (a.sink ? expf(sink - M) : 0.f));
    float *out = a.dst + (int64_t)h * a.dst_s_head + (int64_t)t * a.dst_s_tok;
#pragma unroll
    for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; if (j < KR) out[j] = acc[i] * f * inv; }
}

template <int NL, int NR>
static int launch_latent_attn_tile(const b200_latent_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)a->n_tokens, (unsigned)((a->n_head + LT_HEADS - 1) / LT_HEADS));
    const size_t smem = (size_t)LT_CELLS * (a->kv_rank + a->rot_dim) * 4;
    if (smem > 48 * 1024) B200_CUDA_TRY(cudaFuncSetAttribute(latent_attn_tile_kernel<NL, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    latent_attn_tile_kernel<NL, NR><<<grid, LT_HEADS * 32, smem, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

template <int NL, int NR, int WARPS>
static int launch_latent_attn3(const b200_latent_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)a->n_tokens, (unsigned)a->n_head);
    const size_t smem = ((size_t)WARPS * a->kv_rank + 2 * WARPS) * 4;
    if (smem > 48 * 1024) B200_CUDA_TRY(cudaFuncSetAttribute(latent_attn_kernel<NL, NR, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    latent_attn_kernel<NL, NR, WARPS><<<grid, WARPS * 32, smem, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
template <int NL, int NR>
static int launch_latent_attn2(const b200_latent_attn_args *a, cudaStream_t st) {
    // few (token, head) pairs: 16 warps share the cells of a pair
    if ((int64_t)a->n_tokens * a->n_head < 2 * 148 && a->n_kv > 64) return launch_latent_attn3<NL, NR, 16>(a, st);
    // prompt batches: heads of a token share the staged rows (16-byte copies: rows and the cache base must allow them)
    if (a->n_head >= 2 && (a->kv_rank + a->rot_dim) % 4 == 0 && a->cache_stride % 4 == 0 && ((uintptr_t)a->cache & 15) == 0 &&
        (size_t)LT_CELLS * (a->kv_rank + a->rot_dim) * 4 <= 160 * 1024)
        return launch_latent_attn_tile<NL, NR>(a, st);
    return launch_latent_attn3<NL, NR, 4>(a, st);
}
template <int NL>
static int launch_latent_attn(const b200_latent_attn_args *a, cudaStream_t st) {
    const int nr = (a->rot_dim + 31) / 32;
    if (nr <= 1) return launch_latent_attn2<NL, 1>(a, st);
    if (nr <= 2) return launch_latent_attn2<NL, 2>(a, st);
    return launch_latent_attn2<NL, 4>(a, st);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_op_latent_kv_store(const float *dkv, int64_t dkv_stride, const float *w, const int32_t *pos, const float *freqs, const int32_t *cells,
                                       float *cache, int64_t cache_stride, int32_t kv_rank, int32_t rot_dim, int32_t n_dims, float mscale, float eps,
                                       int32_t n_tokens, b200_stream_t stream) {
    OPX_REQUIRE(dkv && w && pos && freqs && cells && cache, B200_ERR_INVALID, "b200_op_latent_kv_store: NULL argument");
    OPX_REQUIRE(kv_rank > 0 && rot_dim >= 0 && n_dims >= 0 && n_dims % 2 == 0 && n_dims <= rot_dim && cache_stride >= kv_rank + rot_dim && n_tokens >= 0,
                B200_ERR_INVALID, "b200_op_latent_kv_store: bad sizes");
    if (n_tokens == 0) return B200_OK;
    latent_kv_store_kernel<<<(unsigned)n_tokens, 128, 0, (cudaStream_t)stream>>>(dkv, dkv_stride, w, pos, freqs, cells, cache, cache_stride, kv_rank, rot_dim,
                                                                                 n_dims, mscale, eps);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_op_latent_attn(const b200_latent_attn_args *a, b200_stream_t stream) {
    OPX_REQUIRE(a && a->q_lat && a->cache && a->cell_seq && a->cell_pos && a->tok_seq && a->tok_pos && a->dst && (a->q_rot || a->rot_dim == 0), B200_ERR_INVALID,
                "b200_op_latent_attn: NULL argument");
    OPX_REQUIRE(a->kv_rank > 0 && a->kv_rank <= 1024 && a->rot_dim >= 0 && a->rot_dim <= 128 && a->n_head > 0 && a->n_head <= 65535 && a->n_tokens >= 0 && a->n_kv >= 0 &&
                a->cache_stride >= a->kv_rank + a->rot_dim, B200_ERR_UNSUPPORTED, "b200_op_latent_attn: kv_rank <= 1024, rot_dim <= 128, heads <= 65535");
    if (a->n_tokens == 0) return B200_OK;
    const cudaStream_t st = (cudaStream_t)stream;
    const int nl = (a->kv_rank + 31) / 32;
    if (nl <= 2) return launch_latent_attn<2>(a, st);
    if (nl <= 4) return launch_latent_attn<4>(a, st);
    if (nl <= 8) return launch_latent_attn<8>(a, st);
    if (nl <= 16) return launch_latent_attn<16>(a, st);
    return launch_latent_attn<32>(a, st);
}
