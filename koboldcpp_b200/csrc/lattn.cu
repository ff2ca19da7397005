// lattn.cu -- attention over a latent KV cache (include/b200_ggml_ops.h: b200_op_latent_kv_store, b200_op_latent_attn).
//
// A cache row holds kv_rank normalised latent values followed by rot_dim rotated key values; all heads read the same rows.
// With the key up-projection folded into the query (q_lat = W_uk^T q) and the value up-projection applied after the weighted
// sum, one head's work per cell is a dot product over the whole row and an axpy over its first kv_rank values, so the cache is
// streamed once per (token, head group) and never expanded to per-head keys and values in HBM.
// Visibility is decided per (token, cell) from (sequence, position) pairs: no mask tensor is built, uploaded or read.
#include "ops_util.cuh"
#include <cuda_bf16.h>

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
    // a warp looks at 32 cells at a time, one per lane, and then works through the visible ones LA_UNROLL at a time: a cache shared
    // with other sequences costs one ballot per 32 of their cells, not a round of loads
    for (int cb = warp * 32; cb < a.n_kv; cb += WARPS * 32) {
        bool mine = false;
        if (cb + lane < a.n_kv) {
            const int cp = a.cell_pos[cb + lane];
            mine = a.cell_seq[cb + lane] == seq && cp <= pos && cp > lo;
        }
        unsigned rest = __ballot_sync(0xffffffffu, mine);
        while (rest) {
            bool vis[LA_UNROLL];  // warp-uniform
            int cu[LA_UNROLL];
            float rv[LA_UNROLL][NL], rr[LA_UNROLL][NR];
#pragma unroll
            for (int u = 0; u < LA_UNROLL; u++) {
                vis[u] = rest != 0u;
                cu[u] = vis[u] ? cb + __ffs(rest) - 1 : 0;
                rest &= rest - 1;  // 0 stays 0
            }
#pragma unroll
            for (int u = 0; u < LA_UNROLL; u++) {
                if (!vis[u]) continue;
                const float *row = a.cache + (int64_t)cu[u] * a.cache_stride;
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

// Prompt batches with bf16 products: the tensor cores take both contractions (mma.sync.m16n8k16, bf16 in, f32 accumulators).
// One CTA per (16 consecutive tokens of the batch, head).  Its query rows [q_lat | q_rot] sit in shared memory as bf16; the cache
// rows come through in tiles of 16 cells, converted to bf16 on the way in.  The LM_WARPS warps split the long contraction of the
// scores (kv_rank + rot_dim values) by 16-wide steps and add their partial 16 x 16 score tiles through shared memory, so every
// warp then holds the whole tile in accumulator layout; scale, visibility, the running maximum and the exponentials are f32 and
// the same in every warp.  For the second product each warp owns a share of the kv_rank output columns (16-wide column groups
// w, w + LM_WARPS, ...), NJ groups per warp, which keeps the f32 accumulators of a 16 x kv_rank result within the register file.
// A tile none of whose cells is visible to any of the 16 tokens is skipped before it is loaded; rows of free cells are read as zeros
// (their weight is zero, and zero times whatever an unwritten row holds must not reach the sum).
// The rows of the next visible tile are fetched into registers before the current tile is worked on (warp w fetches cells w and
// w + 8, a lane every 32nd float4 of a row: NI = ceil(row / 128 floats) loads per row and lane), so the trip to L2 overlaps the
// tensor-core work instead of standing in front of it.  NI also bounds the column groups per warp: kv_rank / 16 <= 8 NI.
constexpr int LM_TOK = 16, LM_CELLS = 16, LM_WARPS = 8, LM_PT_STRIDE = 48;
__device__ __forceinline__ void lm_ldsm4(unsigned addr, unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lm_ldsm4_t(unsigned addr, unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lm_mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned lm_pack_bf2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned *>(&v);
}

template <int NI>
__global__ void __launch_bounds__(LM_WARPS * 32, NI <= 5 ? 2 : 1) latent_attn_mma_kernel(const b200_latent_attn_args a) {
    extern __shared__ float4 lm_smem4[];
    const int KR = a.kv_rank, RS = KR + a.rot_dim, RS16 = (RS + 15) & ~15, NK = RS16 / 16, NJG = KR / 16;
    const int stride = RS16 * 2 + 16;  // bytes per bf16 row: 8 consecutive rows start in 8 different 16-byte bank groups (ldmatrix)
    unsigned char *qs = reinterpret_cast<unsigned char *>(lm_smem4);  // [LM_TOK][stride]
    unsigned char *ts = qs + LM_TOK * stride;                         // [LM_CELLS][stride]
    float *sp = reinterpret_cast<float *>(ts + LM_CELLS * stride);    // [LM_WARPS][32 lanes][8]: partial score tiles in accumulator layout
    int *tseq = reinterpret_cast<int *>(sp + LM_WARPS * 256), *tpos = tseq + LM_TOK, *tlo = tpos + LM_TOK, *cseq = tlo + LM_TOK, *cpos = cseq + LM_CELLS;
    float *alph = reinterpret_cast<float *>(cpos + LM_CELLS);           // [LM_TOK]: what a row's accumulators are scaled by at this tile; at the end its final weight
    unsigned char *pt = reinterpret_cast<unsigned char *>(alph + LM_TOK);  // [LM_TOK][LM_PT_STRIDE]: the tile's weights as bf16 (the A operand of the second product)
    unsigned *tbits = reinterpret_cast<unsigned *>(pt + LM_TOK * LM_PT_STRIDE);  // one bit per tile of cells: something to see there
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int t0 = blockIdx.x * LM_TOK, h = blockIdx.y;

    if (tid < LM_TOK) {
        const int t = t0 + tid;
        const bool ok = t < a.n_tokens;
        const int p = ok ? a.tok_pos[t] : 0;
        tseq[tid] = ok ? a.tok_seq[t] : -2;  // matches no cell
        tpos[tid] = p;
        tlo[tid] = a.window > 0 ? p - a.window : INT_MIN;
    }
    // queries: warp w stages token rows w and w + 8, four loads in flight per lane
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int i = warp + 8 * r, t = t0 + i;
        const bool ok = t < a.n_tokens;
        const float *ql = a.q_lat + (int64_t)h * a.q_lat_s_head + (int64_t)(ok ? t : 0) * a.q_lat_s_tok;
        const float *qr = a.q_rot ? a.q_rot + (int64_t)h * a.q_rot_s_head + (int64_t)(ok ? t : 0) * a.q_rot_s_tok : a.q_lat;
        for (int j0 = lane; j0 < RS16; j0 += 128) {
            float v[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int j = j0 + 32 * k;
                v[k] = !ok || j >= RS ? 0.f : j < KR ? ql[j] : qr[j - KR];
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int j = j0 + 32 * k;
                if (j < RS16) *reinterpret_cast<__nv_bfloat16 *>(qs + i * stride + j * 2) = __float2bfloat16_rn(v[k]);
            }
        }
    }
    // which tiles hold a cell that one of the 16 tokens sees: one bit per tile, found once, warp w looks at tiles w, w + 8, ...;
    // a lane takes one cell of the tile against 8 of the tokens
    const int n_tiles = (a.n_kv + LM_CELLS - 1) / LM_CELLS;
    for (int i = tid; i < (n_tiles + 31) / 32; i += LM_WARPS * 32) tbits[i] = 0u;
    __syncthreads();
    for (int tile = warp; tile < n_tiles; tile += LM_WARPS) {
        const int c = tile * LM_CELLS + (lane & 15), i0 = (lane >> 4) * 8;
        bool any = false;
        if (c < a.n_kv) {
            const int cs = a.cell_seq[c], cp = a.cell_pos[c];
            if (cs >= 0) {
#pragma unroll
                for (int i = i0; i < i0 + 8; i++) any |= cs == tseq[i] && cp <= tpos[i] && cp > tlo[i];
            }
        }
        if (__ballot_sync(0xffffffffu, any) != 0u && lane == 0) atomicOr(&tbits[tile >> 5], 1u << (tile & 31));
    }
    __syncthreads();

    // ldmatrix lane addresses: matrix mi = lane >> 3, row mr = lane & 7
    const int mi = lane >> 3, mr = lane & 7;
    const unsigned qs_u = (unsigned)__cvta_generic_to_shared(qs), ts_u = (unsigned)__cvta_generic_to_shared(ts);
    const unsigned a_off = (unsigned)(((mi & 1) * 8 + mr) * stride + (mi >> 1) * 16);  // A (queries) and transposed B (values): rows (mi&1)*8.., columns (mi>>1)*8..
    const unsigned k_off = (unsigned)(((mi >> 1) * 8 + mr) * stride + (mi & 1) * 16);  // B (keys): cells (mi>>1)*8.., values (mi&1)*8..

    // softmax bookkeeping: warp w owns token rows 2 w and 2 w + 1, a lane one (row, cell of the tile) pair; m and l of the row are
    // the same in its 16 lanes
    const int my_r = 2 * warp + (lane >> 4), my_u = lane & 15;
    const int my_seq = tseq[my_r], my_pos = tpos[my_r], my_lo = tlo[my_r];
    const int sp_off = ((my_r & 7) * 4 + ((my_u & 7) >> 1)) * 8 + (my_u >> 3) * 4 + (my_r >> 3) * 2 + (my_u & 1);  // the pair's place in a partial tile
    const unsigned pt_u = (unsigned)__cvta_generic_to_shared(pt);
    const unsigned p_off = (unsigned)(((mi & 1) * 8 + mr) * LM_PT_STRIDE + (mi >> 1) * 16);
    float m_row = -INFINITY, l_row = 0.f;
    constexpr int NJ = NI;
    float o[NJ][2][4];
#pragma unroll
    for (int jj = 0; jj < NJ; jj++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[jj][0][e] = o[jj][1][e] = 0.f;
    const int RS4 = RS / 4, RS16_4 = RS16 / 4;

    // the first tile from `from` on with a cell that one of the 16 tokens sees (n_kv: none)
    auto next_tile = [&](int from) {
        int tile = from / LM_CELLS;
        while (tile < n_tiles) {
            const unsigned rest = tbits[tile >> 5] >> (tile & 31);
            if (rest) return (tile + __ffs(rest) - 1) * LM_CELLS;
            tile = (tile | 31) + 1;
        }
        return a.n_kv;
    };
    float4 pf[2][NI];
    int pf_seq = -1, pf_pos = -1;  // threads < LM_CELLS: the cell's owner and position
    auto fetch = [&](int c0) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int c = c0 + warp + 8 * r;
            const bool ok = c < a.n_kv && a.cell_seq[c] >= 0;
            const float4 *row = reinterpret_cast<const float4 *>(a.cache + (int64_t)(ok ? c : 0) * a.cache_stride);
#pragma unroll
            for (int i = 0; i < NI; i++) {
                const int j = lane + 32 * i;
                pf[r][i] = ok && j < RS4 ? row[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (tid < LM_CELLS) {
            const int c = c0 + tid;
            pf_seq = c < a.n_kv ? a.cell_seq[c] : -1;
            pf_pos = c < a.n_kv ? a.cell_pos[c] : -1;
        }
    };
    int c0 = next_tile(0);
    if (c0 < a.n_kv) fetch(c0);
    while (c0 < a.n_kv) {
        __syncthreads();  // the previous tile, its scores and its cell table have been read
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int i = 0; i < NI; i++) {
                const int j = lane + 32 * i;
                if (j < RS16_4)
                    *reinterpret_cast<uint2 *>(ts + (warp + 8 * r) * stride + j * 8) = make_uint2(lm_pack_bf2(pf[r][i].x, pf[r][i].y), lm_pack_bf2(pf[r][i].z, pf[r][i].w));
            }
        if (tid < LM_CELLS) { cseq[tid] = pf_seq; cpos[tid] = pf_pos; }
        __syncthreads();
        c0 = next_tile(c0 + LM_CELLS);
        if (c0 < a.n_kv) fetch(c0);  // in flight while this tile is worked on
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        for (int ks = warp; ks < NK; ks += LM_WARPS) {
            unsigned qa[4], b0, b1, b2, b3;
            lm_ldsm4(qs_u + a_off + ks * 32, qa[0], qa[1], qa[2], qa[3]);
            lm_ldsm4(ts_u + k_off + ks * 32, b0, b1, b2, b3);
            lm_mma_bf16(s[0], qa, b0, b1);  // cells 0-7
            lm_mma_bf16(s[1], qa, b2, b3);  // cells 8-15
        }
        {
            float4 *mine = reinterpret_cast<float4 *>(sp + (warp * 32 + lane) * 8);
            mine[0] = make_float4(s[0][0], s[0][1], s[0][2], s[0][3]);
            mine[1] = make_float4(s[1][0], s[1][1], s[1][2], s[1][3]);
        }
        __syncthreads();
        {
            float sv = 0.f;
#pragma unroll
            for (int w = 0; w < LM_WARPS; w++) sv += sp[w * 256 + sp_off];
            const int cp = cpos[my_u];
            const bool vis = cseq[my_u] == my_seq && cp <= my_pos && cp > my_lo;
            sv = vis ? sv * a.scale : -INFINITY;
            float mx = sv;
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));  // over the row's 16 lanes
            const float mn = fmaxf(m_row, mx);
            const bool none = mn == -INFINITY;  // nothing seen so far by this row
            const float al = none ? 1.0f : expf(m_row - mn), pw = none ? 0.f : expf(sv - mn);
            float ps = pw;
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            l_row = l_row * al + ps;
            m_row = mn;
            *reinterpret_cast<__nv_bfloat16 *>(pt + my_r * LM_PT_STRIDE + my_u * 2) = __float2bfloat16_rn(pw);
            if (my_u == 0) alph[my_r] = al;
        }
        __syncthreads();
        unsigned pa[4];
        lm_ldsm4(pt_u + p_off, pa[0], pa[1], pa[2], pa[3]);
        const float alpha[2] = {alph[g], alph[g + 8]};
        const bool rescale = __any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f);
#pragma unroll
        for (int jj = 0; jj < NJ; jj++) {
            const int j = warp + jj * LM_WARPS;
            if (j >= NJG) break;
            if (rescale) {
#pragma unroll
                for (int half = 0; half < 2; half++) { o[jj][half][0] *= alpha[0]; o[jj][half][1] *= alpha[0]; o[jj][half][2] *= alpha[1]; o[jj][half][3] *= alpha[1]; }
            }
            unsigned b0, b1, b2, b3;
            lm_ldsm4_t(ts_u + a_off + j * 32, b0, b1, b2, b3);
            lm_mma_bf16(o[jj][0], pa, b0, b1);  // columns 16 j .. 16 j + 7
            lm_mma_bf16(o[jj][1], pa, b2, b3);  // columns 16 j + 8 .. 16 j + 15
        }
    }
    __syncthreads();  // the last tile's scale factors have been read
    if (my_u == 0) {
        const float sink = a.sink ? a.sink[h] : -INFINITY;
        const float M = fmaxf(m_row, sink);
        const float f = m_row == -INFINITY ? 0.f : expf(m_row - M);
        const float den = l_row * f + (a.sink ? expf(sink - M) : 0.f);
        alph[my_r] = den > 0.f ? f / den : 0.f;
    }
    __syncthreads();
    const float w[2] = {alph[g], alph[g + 8]};
#pragma unroll
    for (int jj = 0; jj < NJ; jj++) {
        const int j = warp + jj * LM_WARPS;
        if (j >= NJG) break;
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            const int t = t0 + g + 8 * hh;
            if (t >= a.n_tokens) continue;
            float *out = a.dst + (int64_t)h * a.dst_s_head + (int64_t)t * a.dst_s_tok + 16 * j + 2 * t4;
            out[0] = o[jj][0][2 * hh] * w[hh]; out[1] = o[jj][0][2 * hh + 1] * w[hh];
            out[8] = o[jj][1][2 * hh] * w[hh]; out[9] = o[jj][1][2 * hh + 1] * w[hh];
        }
    }
}

static size_t latent_attn_mma_smem(const b200_latent_attn_args *a) {
    const int rs16 = (a->kv_rank + a->rot_dim + 15) & ~15;
    return (size_t)(LM_TOK + LM_CELLS) * (rs16 * 2 + 16) + (size_t)LM_WARPS * 256 * 4 + (3 * LM_TOK + 2 * LM_CELLS + LM_TOK) * 4 + LM_TOK * LM_PT_STRIDE +
           (size_t)(((a->n_kv + LM_CELLS - 1) / LM_CELLS + 31) / 32) * 4;
}
template <int NI>
static int launch_latent_attn_mma2(const b200_latent_attn_args *a, cudaStream_t st) {
    const dim3 grid((unsigned)((a->n_tokens + LM_TOK - 1) / LM_TOK), (unsigned)a->n_head);
    const size_t smem = latent_attn_mma_smem(a);
    if (smem > 48 * 1024) B200_CUDA_TRY(cudaFuncSetAttribute(latent_attn_mma_kernel<NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    latent_attn_mma_kernel<NI><<<grid, LM_WARPS * 32, smem, st>>>(*a);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
// bf16 products were asked for, there are enough tokens to fill 16-row tiles, and the sizes fit the 16-wide fragments and 16-byte copies
static bool latent_attn_mma_ok(const b200_latent_attn_args *a) {
    return a->bf16_products && a->n_tokens >= LM_TOK && a->kv_rank % 16 == 0 && (a->kv_rank + a->rot_dim) % 4 == 0 && a->cache_stride % 4 == 0 &&
           ((uintptr_t)a->cache & 15) == 0 && latent_attn_mma_smem(a) <= 200 * 1024;
}
static int launch_latent_attn_mma(const b200_latent_attn_args *a, cudaStream_t st) {
    const int ni = (((a->kv_rank + a->rot_dim + 15) & ~15) + 127) / 128;  // <= 9 for kv_rank <= 1024, rot_dim <= 128
    if (ni <= 1) return launch_latent_attn_mma2<1>(a, st);
    if (ni <= 2) return launch_latent_attn_mma2<2>(a, st);
    if (ni <= 3) return launch_latent_attn_mma2<3>(a, st);
    if (ni <= 5) return launch_latent_attn_mma2<5>(a, st);
    if (ni <= 7) return launch_latent_attn_mma2<7>(a, st);
    return launch_latent_attn_mma2<9>(a, st);
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
    if (latent_attn_mma_ok(a)) return launch_latent_attn_mma(a, st);
    const int nl = (a->kv_rank + 31) / 32;
    if (nl <= 2) return launch_latent_attn<2>(a, st);
    if (nl <= 4) return launch_latent_attn<4>(a, st);
    if (nl <= 8) return launch_latent_attn<8>(a, st);
    if (nl <= 16) return launch_latent_attn<16>(a, st);
    return launch_latent_attn<32>(a, st);
}
