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

// One CTA per (token, head); warps stride over the cells, each keeping an online softmax and a latent accumulator that are
// merged through shared memory at the end.  NL = ceil(kv_rank / 32), NR = ceil(rot_dim / 32): values per lane.
constexpr int LA_WARPS = 4;
template <int NL, int NR>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attn_kernel(const b200_latent_attn_args a) {
    extern __shared__ float smem[];  // [LA_WARPS][kv_rank] accumulators, then m[LA_WARPS], l[LA_WARPS]
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
    for (int c = warp; c < a.n_kv; c += LA_WARPS) {
        const int cp = a.cell_pos[c];
        if (a.cell_seq[c] != seq || cp > pos || cp <= lo) continue;  // warp-uniform
        const float *row = a.cache + (int64_t)c * a.cache_stride;
        float rv[NL], s = 0.f;
#pragma unroll
        for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; rv[i] = j < KR ? row[j] : 0.f; s += q1[i] * rv[i]; }
#pragma unroll
        for (int i = 0; i < NR; i++) { const int j = lane + 32 * i; s += q2[i] * (j < R ? row[KR + j] : 0.f); }
        s = warp_sum(s);
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), p = expf(s - mn);  // m = -inf at the first cell: corr = 0
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < NL; i++) acc[i] = acc[i] * corr + p * rv[i];
        m = mn;
    }
    float *sacc = smem + (size_t)warp * KR, *sm = smem + (size_t)LA_WARPS * KR, *sl = sm + LA_WARPS;
#pragma unroll
    for (int i = 0; i < NL; i++) { const int j = lane + 32 * i; if (j < KR) sacc[j] = acc[i]; }
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
    __syncthreads();
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    float M = sink;
#pragma unroll
    for (int w = 0; w < LA_WARPS; w++) M = fmaxf(M, sm[w]);
    float L = a.sink ? expf(sink - M) : 0.f, f[LA_WARPS];
#pragma unroll
    for (int w = 0; w < LA_WARPS; w++) { f[w] = sm[w] == -INFINITY ? 0.f : expf(sm[w] - M); L += sl[w] * f[w]; }
    const float inv = 1.0f / L;
    float *out = a.dst + (int64_t)h * a.dst_s_head + (int64_t)t * a.dst_s_tok;
    for (int j = threadIdx.x; j < KR; j += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < LA_WARPS; w++) o += smem[(size_t)w * KR + j] * f[w];
        out[j] = o * inv;
    }
}

template <int NL>
static int launch_latent_attn(const b200_latent_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)a->n_tokens, (unsigned)a->n_head);
    const size_t smem = ((size_t)LA_WARPS * a->kv_rank + 2 * LA_WARPS) * 4;
    const int nr = (a->rot_dim + 31) / 32;
#define B200_LA_LAUNCH(NR)                                                                                                              \
    do {                                                                                                                                \
        if (smem > 48 * 1024) B200_CUDA_TRY(cudaFuncSetAttribute(latent_attn_kernel<NL, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        latent_attn_kernel<NL, NR><<<grid, LA_WARPS * 32, smem, st>>>(*a);                                                              \
    } while (0)
    if (nr <= 1) B200_LA_LAUNCH(1); else if (nr <= 2) B200_LA_LAUNCH(2); else B200_LA_LAUNCH(4);
#undef B200_LA_LAUNCH
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
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
