// host_genesun.cu -- the Genesun architecture for the decoder of host_llama.cu: where its tensors go and the graph of one
// batch step.  The decoder owns the model object, the sequence cache, the inputs and the step; this file adds no loop of its own.
//
// A Genesun model is a stack of layers of two kinds, each with its own shapes (b200_layer_params):
//   * latent attention: queries through a normalised latent, one normalised latent per token for keys and values plus one
//     rotated key part shared by all heads, softmax with a per-head sink, an output gate; a layer may read another layer's cache;
//   * mLSTM: a matrix memory per head with exponential gating;
// every sublayer's result passes a sigmoid gate and a layer norm before it is added to the residual, the feed-forward uses the
// PolyNorm activation, and the input of layer i + 1 is a learned weighted sum of the embedding and the results of layers 0 .. i.
//
// Graph choices: all projections that read one normalised activation are ONE matmul over row-concatenated weights (set_tensor
// appends the parts in a fixed order); the key up-projection is folded into the query (per-head matmul over the transposed
// weight, laid out at upload) and the value up-projection follows the attention, so the attention kernel streams the latent
// cache rows only; the layer results are written straight into one stacked tensor that the weighted sum reads.
#include "host_model.h"

namespace {

struct GsLayer {
    ggml_tensor *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr, *rg1b = nullptr, *rg2b = nullptr, *dwa = nullptr;
    ggml_tensor *proj1 = nullptr, *proj2 = nullptr;  // fused rows over norm1(x) / norm2(x)
    ggml_tensor *dq_norm = nullptr, *uq = nullptr, *dkv_norm = nullptr, *uk_t = nullptr, *uv = nullptr, *sink = nullptr, *wo = nullptr;
    ggml_tensor *mnorm = nullptr, *ib = nullptr, *fb = nullptr;
    ggml_tensor *down = nullptr, *act = nullptr;
    ggml_tensor *freqs = nullptr;
    float mscale = 1.0f;
    ggml_tensor *cache = nullptr;  // latent attention: [kv_rank + rot_dim, n_ctx] f32 (the owner's tensor when kv_from >= 0)
    ggml_tensor *state = nullptr;  // mLSTM: [state floats, n_seq_max] f32
    ggml_tensor *store_node = nullptr;  // this graph's cache-store node (readers of the cache depend on it)
};
struct GsData {
    std::vector<GsLayer> layers;
    ggml_tensor *embed = nullptr, *final_norm = nullptr, *head = nullptr;
};
GsData *gs(b200_llama *m) { return (GsData *)m->arch_data.get(); }

// rows of the fused projections, in upload order
struct Part { const char *leaf; int64_t rows; };
int parts_proj1(const b200_llama *m, const b200_layer_params &lp, Part out[8]) {
    const int64_t W = m->hp.n_embd;
    int n = 0;
    if (lp.mixer == B200_MIXER_LATENT_ATTENTION) {
        out[n++] = {"mix.dq", lp.q_rank};
        if (lp.kv_from < 0) out[n++] = {"mix.dkv", (int64_t)lp.kv_rank + lp.rot_dim};
        out[n++] = {"mix.g", (int64_t)lp.heads * lp.vdim};
    } else {
        out[n++] = {"mix.q", (int64_t)lp.heads * lp.dim};
        out[n++] = {"mix.k", (int64_t)lp.heads * lp.dim};
        out[n++] = {"mix.v", (int64_t)lp.heads * lp.vdim};
        out[n++] = {"mix.g", (int64_t)lp.heads * lp.vdim};
        out[n++] = {"mix.i", lp.heads};
        out[n++] = {"mix.f", lp.heads};
    }
    out[n++] = {"rg1", W};
    return n;
}
int parts_proj2(const b200_llama *m, const b200_layer_params &lp, Part out[8]) {
    if (lp.mlp == B200_MLP_NONE) return 0;
    out[0] = {"mlp.up", lp.ff};
    out[1] = {"rg2", m->hp.n_embd};
    return 2;
}
int64_t part_offset(const Part *p, int n, const char *leaf, int64_t *total) {
    int64_t off = 0, found = -1;
    for (int i = 0; i < n; i++) { if (!strcmp(p[i].leaf, leaf)) found = off; off += p[i].rows; }
    if (total) *total = off;
    return found;
}

// "l<i>.<leaf>" -> i, leaf
bool split_name(const char *name, int *il, const char **leaf) {
    if (name[0] != 'l' || name[1] < '0' || name[1] > '9') return false;
    char *end = nullptr;
    const long v = strtol(name + 1, &end, 10);
    if (!end || *end != '.') return false;
    *il = (int)v;
    *leaf = end + 1;
    return true;
}

int gs_place_tensor(b200_llama *m, const char *name, int type, int64_t ne0, int64_t ne1, int64_t ne2, const void *data) {
    int il = -1;
    const char *leaf = nullptr;
    if (!split_name(name, &il, &leaf)) return upload_tensor(m, name, type, ne0, ne1, ne2, data);
    LL_REQUIRE(il >= 0 && il < m->hp.n_layer, B200_ERR_INVALID, "b200_llama_set_tensor: %s names a layer outside 0..%d", name, m->hp.n_layer - 1);
    const b200_layer_params &lp = m->layer_hp[(size_t)il];
    LL_REQUIRE(lp.mixer != 0, B200_ERR_INVALID, "b200_llama_set_tensor: %s before b200_llama_set_layer(%d)", name, il);
    const TypeTraits tt = type_traits(type);
    LL_REQUIRE(tt.blck == 1 && ne2 == 1, B200_ERR_UNSUPPORTED, "b200_llama_set_tensor: %s: dense 1-D / 2-D tensors only", name);
    if (lp.mixer == B200_MIXER_LATENT_ATTENTION && !strcmp(leaf, "mix.uk")) {
        // [kv_rank, heads * dim] -> per head the transpose [dim, kv_rank]: the contraction with the query runs over dim
        const int64_t KR = lp.kv_rank, D = lp.dim, H = lp.heads;
        LL_REQUIRE(ne0 == KR && ne1 == H * D, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0,
                   (long long)(H * D), (long long)KR);
        const size_t es = (size_t)tt.size;
        std::vector<char> t((size_t)(KR * D * H) * es);
        const char *src = (const char *)data;
        for (int64_t h = 0; h < H; h++)
            for (int64_t d = 0; d < D; d++)
                for (int64_t r = 0; r < KR; r++) memcpy(&t[(size_t)((h * KR + r) * D + d) * es], src + (size_t)((h * D + d) * KR + r) * es, es);
        return upload_tensor(m, (std::string(name) + "_t").c_str(), type, D, KR, H, t.data());
    }
    for (int which = 0; which < 2; which++) {
        Part parts[8];
        const int n = which ? parts_proj2(m, lp, parts) : parts_proj1(m, lp, parts);
        int64_t total = 0;
        const int64_t off = part_offset(parts, n, leaf, &total);
        if (off < 0) continue;
        int64_t rows = 0;
        for (int i = 0; i < n; i++) if (!strcmp(parts[i].leaf, leaf)) rows = parts[i].rows;
        LL_REQUIRE(ne0 == m->hp.n_embd && ne1 == rows, B200_ERR_INVALID, "b200_llama_set_tensor: %s is [%lld, %lld], expected [%lld, %lld]", name, (long long)ne1, (long long)ne0,
                   (long long)rows, (long long)m->hp.n_embd);
        const std::string fused = "l" + std::to_string(il) + (which ? ".proj2" : ".proj1");
        ggml_tensor *f = find_w(m, fused);
        if (!f) {
            m->weight_pool.emplace_back();
            f = &m->weight_pool.back();
            memset(f, 0, sizeof(*f));
            set_shape(f, type, ne0, total, 1, 1);
            snprintf(f->name, sizeof(f->name), "%s", fused.c_str());
            if (!alloc_in_buft(m, m->buft, f, GGML_BACKEND_BUFFER_USAGE_WEIGHTS)) {
                m->weight_pool.pop_back();
                b200::set_error("b200_llama_set_tensor: out of device memory for %s (%zu bytes)", fused.c_str(), nbytes(f));
                return B200_ERR_NOMEM;
            }
            m->weights[fused] = f;
            m->weight_bytes += (int64_t)nbytes(f);
        }
        LL_REQUIRE(f->type == type, B200_ERR_INVALID, "b200_llama_set_tensor: %s: the parts of %s must have one type", name, fused.c_str());
        LL_REQUIRE(m->weights.find(name) == m->weights.end(), B200_ERR_INVALID, "b200_llama_set_tensor: duplicate tensor %s", name);
        f->buffer->iface.set_tensor(f->buffer, f, data, (size_t)off * f->nb[1], (size_t)rows * f->nb[1]);
        m->weights[name] = f;  // marks the part as present
        return B200_OK;
    }
    return upload_tensor(m, name, type, ne0, ne1, ne2, data);
}

// per-pair rotation frequencies with YaRN's blend of extrapolated and interpolated frequencies, in double, rounded once
void rope_freqs(const b200_layer_params &lp, std::vector<float> &f, float *mscale) {
    const int dims = lp.rope_dims;
    f.resize((size_t)(dims / 2));
    *mscale = 1.0f;
    const double base = lp.rope_base;
    const bool yarn = lp.yarn_factor > 0.0f && lp.yarn_factor != 1.0f;
    double lo = 0, hi = 0;
    if (yarn) {
        auto corr = [&](double turns) { return dims * log((double)lp.yarn_original / (2.0 * M_PI * turns)) / (2.0 * log(base)); };
        lo = fmax(floor(corr(lp.yarn_fast)), 0.0);
        hi = fmin(ceil(corr(lp.yarn_slow)), (double)dims - 1.0);
        *mscale = (float)(0.1 * log((double)lp.yarn_factor) + 1.0);
    }
    for (int i = 0; i < dims / 2; i++) {
        double fi = pow(base, -2.0 * i / dims);
        if (yarn) {
            const double ramp = fmin(fmax((i - lo) / fmax(hi - lo, 0.001), 0.0), 1.0);
            fi = fi / lp.yarn_factor * ramp + fi * (1.0 - ramp);
        }
        f[(size_t)i] = (float)fi;
    }
}

int gs_finalize(b200_llama *m) {
    const b200_llama_params &hp = m->hp;
    m->arch_data = std::shared_ptr<void>(new GsData(), [](void *p) { delete (GsData *)p; });
    GsData *g = gs(m);
    LL_REQUIRE(m->run_layer.empty(), B200_ERR_UNSUPPORTED, "b200_llama_finalize: this architecture runs every layer once, in order");
    g->layers.resize((size_t)hp.n_layer);
    g->embed = find_w(m, "embed"); g->final_norm = find_w(m, "final.norm"); g->head = find_w(m, "head");
    LL_REQUIRE(g->embed && g->final_norm && g->head, B200_ERR_INVALID, "b200_llama_finalize: embed / final.norm / head missing");
    LL_REQUIRE(g->embed->ne[0] == hp.n_embd && g->embed->ne[1] == hp.n_vocab && g->head->ne[0] == hp.n_embd && g->head->ne[1] == hp.n_vocab, B200_ERR_INVALID,
               "b200_llama_finalize: embed / head do not fit width %d and vocabulary %d", hp.n_embd, hp.n_vocab);
    for (int il = 0; il < hp.n_layer; il++) {
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        GsLayer &L = g->layers[(size_t)il];
        const std::string pre = "l" + std::to_string(il) + ".";
        auto need = [&](const char *leaf, int64_t ne0, int64_t ne1, int64_t ne2 = 1) -> ggml_tensor * {
            ggml_tensor *t = find_w(m, pre + leaf);
            if (!t) { b200::set_error("b200_llama_finalize: tensor %s%s missing", pre.c_str(), leaf); return nullptr; }
            if (t->ne[0] != ne0 || t->ne[1] != ne1 || t->ne[2] != ne2) {
                b200::set_error("b200_llama_finalize: tensor %s%s has shape [%lld, %lld, %lld], the layer's sizes give [%lld, %lld, %lld]", pre.c_str(), leaf, (long long)t->ne[2],
                                (long long)t->ne[1], (long long)t->ne[0], (long long)ne2, (long long)ne1, (long long)ne0);
                return nullptr;
            }
            return t;
        };
#define GS_NEED(dst, ...) do { dst = need(__VA_ARGS__); if (!(dst)) return B200_ERR_INVALID; } while (0)
        LL_REQUIRE(lp.mixer == B200_MIXER_LATENT_ATTENTION || lp.mixer == B200_MIXER_MLSTM, B200_ERR_INVALID, "b200_llama_finalize: layer %d has no mixer (b200_llama_set_layer)", il);
        LL_REQUIRE(lp.heads > 0 && lp.dim > 0 && lp.vdim > 0, B200_ERR_INVALID, "b200_llama_finalize: layer %d: heads, dim, vdim must be positive", il);
        const int64_t W = hp.n_embd, H = lp.heads, D = lp.dim, V = lp.vdim;
        GS_NEED(L.norm1, "norm1", W, 1); GS_NEED(L.norm1b, "norm1b", W, 1); GS_NEED(L.rg1b, "rg1.b", W, 1); GS_NEED(L.dwa, "dwa", il + 2, 1);
        Part parts[8];
        int np = parts_proj1(m, lp, parts);
        int64_t total = 0;
        part_offset(parts, np, "", &total);
        for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
        GS_NEED(L.proj1, "proj1", W, total);
        if (lp.mixer == B200_MIXER_LATENT_ATTENTION) {
            const int64_t R = lp.rot_dim, KR = lp.kv_rank, QR = lp.q_rank;
            LL_REQUIRE(KR > 0 && QR > 0 && R >= 0 && lp.rope_dims >= 0 && lp.rope_dims % 2 == 0 && lp.rope_dims <= R && (lp.rope_dims == 0 || lp.rope_base > 0.0f), B200_ERR_INVALID,
                       "b200_llama_finalize: layer %d: latent sizes / rotation do not fit", il);
            LL_REQUIRE(KR <= 1024 && R <= 128, B200_ERR_UNSUPPORTED, "b200_llama_finalize: layer %d: kv_rank <= 1024 and rot_dim <= 128", il);
            GS_NEED(L.dq_norm, "mix.dq.norm", QR, 1); GS_NEED(L.uq, "mix.uq", QR, H * (D + R)); GS_NEED(L.uk_t, "mix.uk_t", D, KR, H); GS_NEED(L.uv, "mix.uv", KR, H * V);
            GS_NEED(L.sink, "mix.sink", H, 1); GS_NEED(L.wo, "mix.o", H * V, W);
            std::vector<float> f;
            rope_freqs(lp, f, &L.mscale);
            if (f.empty()) f.push_back(0.0f);
            const std::string fname = pre + "rope_freqs";
            const int rc = upload_tensor(m, fname.c_str(), GGML_TYPE_F32, (int64_t)f.size(), 1, 1, f.data());
            if (rc != B200_OK) return rc;
            L.freqs = find_w(m, fname);
            if (lp.kv_from < 0) {
                GS_NEED(L.dkv_norm, "mix.dkv.norm", KR, 1);
                L.cache = new_device_tensor(m, (pre + "cache").c_str(), GGML_TYPE_F32, KR + R, hp.n_ctx, true);
                LL_REQUIRE(L.cache, B200_ERR_NOMEM, "b200_llama_finalize: out of device memory for the cache of layer %d", il);
                m->kv_bytes += (int64_t)nbytes(L.cache);
            } else {
                LL_REQUIRE(lp.kv_from < il, B200_ERR_INVALID, "b200_llama_finalize: layer %d reads the cache of layer %d, which does not come before it", il, lp.kv_from);
                const b200_layer_params &o = m->layer_hp[(size_t)lp.kv_from];
                LL_REQUIRE(o.mixer == B200_MIXER_LATENT_ATTENTION && o.kv_from < 0 && o.kv_rank == lp.kv_rank && o.rot_dim == lp.rot_dim, B200_ERR_INVALID,
                           "b200_llama_finalize: layer %d cannot read the cache of layer %d (not a latent-attention layer with its own cache of the same shape)", il, lp.kv_from);
                L.cache = g->layers[(size_t)lp.kv_from].cache;
            }
        } else {
            LL_REQUIRE(lp.gate_cap > 0.0f && D <= 512, B200_ERR_INVALID, "b200_llama_finalize: layer %d: gate_cap must be positive and dim <= 512", il);
            GS_NEED(L.mnorm, "mix.norm", H * V, 1); GS_NEED(L.ib, "mix.i.b", H, 1); GS_NEED(L.fb, "mix.f.b", H, 1); GS_NEED(L.wo, "mix.o", H * V, W);
            L.state = new_device_tensor(m, (pre + "state").c_str(), GGML_TYPE_F32, b200_mlstm_state_floats((int32_t)H, (int32_t)D, (int32_t)V), hp.n_seq_max, true);
            LL_REQUIRE(L.state, B200_ERR_NOMEM, "b200_llama_finalize: out of device memory for the state of layer %d", il);
            m->kv_bytes += (int64_t)nbytes(L.state);
        }
        if (lp.mlp != B200_MLP_NONE) {
            LL_REQUIRE(lp.mlp == B200_MLP_DENSE_POLYNORM && lp.ff > 0, B200_ERR_UNSUPPORTED, "b200_llama_finalize: layer %d: unknown feed-forward kind", il);
            GS_NEED(L.norm2, "norm2", W, 1); GS_NEED(L.norm2b, "norm2b", W, 1); GS_NEED(L.rg2b, "rg2.b", W, 1);
            np = parts_proj2(m, lp, parts);
            for (int i = 0; i < np; i++) LL_REQUIRE(find_w(m, pre + parts[i].leaf), B200_ERR_INVALID, "b200_llama_finalize: tensor %s%s missing", pre.c_str(), parts[i].leaf);
            GS_NEED(L.proj2, "proj2", W, (int64_t)lp.ff + W);
            GS_NEED(L.down, "mlp.down", lp.ff, W); GS_NEED(L.act, "mlp.act", 4, 1);
        }
#undef GS_NEED
    }
    return B200_OK;
}

// ------------------------------------------------------------------------------------------------ graph of one batch step
enum { R_STACK = 0, R_EVEN = 1, R_ODD = 2, R_TAIL = 3 };

int gs_build(b200_llama *m, const BatchShape &bs) {
    const b200_llama_params &hp = m->hp;
    GsData *g = gs(m);
    const int64_t T = bs.n_tokens, W = hp.n_embd, NL = hp.n_layer;
    const float eps = hp.rms_eps;
    m->arena.reset();
    Builder b;
    b.arena = &m->arena;
    for (Bump &r : m->regions) r.off = 0;
    auto input_view = [&](const ggml_tensor &base, int64_t ne0, int64_t ne1 = 1) {
        ggml_tensor *t = m->arena.get();
        *t = base;
        set_shape(t, base.type, ne0, ne1, 1, 1);
        return t;
    };
    ggml_tensor *tokens = input_view(m->inp_tokens, T), *pos = input_view(m->inp_pos, T), *cells = input_view(m->inp_cells, T), *tok_seq = input_view(m->inp_tok_seq, T);
    ggml_tensor *cell_seq = input_view(m->inp_cell_seq, bs.n_kv), *cell_pos = input_view(m->inp_cell_pos, bs.n_kv), *seq_info = input_view(m->inp_seq_info, bs.n_seq, 4);

    auto norm = [&](ggml_tensor *dst, ggml_tensor *x, ggml_tensor *w, int kind, int64_t w_period = 1, ggml_tensor *gate = nullptr, ggml_tensor *gate_bias = nullptr,
                    ggml_tensor *res = nullptr) {
        if (!dst) dst = b.alloc_result(GGML_TYPE_F32, x->ne[0], x->ne[1], x->ne[2], 1);
        b.ext(dst, B200_EXT_NORM, {x, w, gate, gate_bias, res});
        dst->op_params[2] = kind; Builder::set_f(dst, 3, eps); dst->op_params[4] = (int32_t)w_period;
        return dst;
    };
    auto sigmoid_mul = [&](ggml_tensor *a, ggml_tensor *gate) {
        return b.ext(b.alloc_result(GGML_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], 1), B200_EXT_SIGMOID_MUL, {a, gate});
    };

    b.bump = &m->regions[R_STACK];
    ggml_tensor *stack = b.alloc_result(GGML_TYPE_F32, W, T, NL + 1);  // the embedding output and every layer's result
    auto slice = [&](int64_t j) { return b.result_at(stack, (size_t)j * stack->nb[2], GGML_TYPE_F32, W, T); };
    ggml_tensor *x = b.op(slice(0), GGML_OP_GET_ROWS, g->embed, tokens);

    for (int il = 0; il < NL; il++) {
        const b200_layer_params &lp = m->layer_hp[(size_t)il];
        GsLayer &L = g->layers[(size_t)il];
        b.bump = &m->regions[(il & 1) ? R_ODD : R_EVEN];
        b.bump->off = 0;
        const int64_t H = lp.heads, D = lp.dim, V = lp.vdim;
        ggml_tensor *h = norm(nullptr, x, L.norm1, B200_NORM_LAYER);
        ggml_tensor *P = b.mul_mat(L.proj1, h);
        Part parts[8];
        const int np = parts_proj1(m, lp, parts);
        auto part = [&](const char *leaf, int64_t rows) { return b.view_2d(P, rows, T, P->nb[1], (size_t)part_offset(parts, np, leaf, nullptr) * 4); };
        ggml_tensor *og;  // the gated mixer output in front of W_o, [H * V, T]
        if (lp.mixer == B200_MIXER_LATENT_ATTENTION) {
            const int64_t R = lp.rot_dim, KR = lp.kv_rank;
            ggml_tensor *cq = norm(nullptr, part("mix.dq", lp.q_rank), L.dq_norm, B200_NORM_RMS);
            ggml_tensor *q = b.mul_mat(L.uq, cq);  // [H * (D + R), T], per head [D unrotated | R rotated]
            ggml_tensor *q_rot = nullptr;
            if (R > 0) {
                ggml_tensor *qr = b.view_3d(q, R, H, T, (size_t)(D + R) * 4, q->nb[1], (size_t)D * 4);
                q_rot = b.view_3d(q, R, H, T, (size_t)(D + R) * 4, q->nb[1], (size_t)D * 4);
                b.ext(q_rot, B200_EXT_ROPE_TABLE, {qr, pos, L.freqs});  // in place
                q_rot->op_params[2] = lp.rope_dims; Builder::set_f(q_rot, 3, L.mscale); q_rot->op_params[4] = 0;
            }
            if (lp.kv_from < 0) {
                ggml_tensor *st = b.view_2d(L.cache, KR + R, hp.n_ctx, L.cache->nb[1], 0);
                b.ext(st, B200_EXT_LATENT_KV_STORE, {part("mix.dkv", KR + R), L.dkv_norm, pos, L.freqs, cells, L.cache});
                st->op_params[2] = (int32_t)KR; Builder::set_f(st, 3, eps); Builder::set_f(st, 4, L.mscale); st->op_params[5] = lp.rope_dims;
                L.store_node = st;
            } else {
                L.store_node = g->layers[(size_t)lp.kv_from].store_node;
            }
            ggml_tensor *q_nope = b.view_3d(q, D, T, H, q->nb[1], (size_t)(D + R) * 4, 0);         // [D, T, H]
            ggml_tensor *q_lat = b.permute(b.mul_mat(L.uk_t, q_nope), 0, 2, 1, 3);               // [KR, T, H] seen as [KR, H, T]
            ggml_tensor *o_lat = b.alloc_result(GGML_TYPE_F32, KR, T, H);
            b.ext(o_lat, B200_EXT_LATENT_ATTN, {q_lat, q_rot, L.store_node, L.sink, tok_seq, pos, cell_seq, cell_pos});
            o_lat->op_params[2] = (int32_t)KR; Builder::set_f(o_lat, 3, lp.scale); o_lat->op_params[4] = lp.window;
            o_lat->op_params[5] = L.uk_t->type == GGML_TYPE_BF16;  // bf16 weights: the attention products of a prompt batch may be bf16 as well
            ggml_tensor *uv3 = b.view_3d(L.uv, KR, V, H, L.uv->nb[1], L.uv->nb[1] * (size_t)V, 0);
            ggml_tensor *o = b.permute(b.mul_mat(uv3, o_lat), 0, 2, 1, 3);                        // [V, T, H] seen as [V, H, T]
            ggml_tensor *gate = b.view_3d(P, V, H, T, (size_t)V * 4, P->nb[1], (size_t)part_offset(parts, np, "mix.g", nullptr) * 4);
            og = b.reshape(sigmoid_mul(o, gate), H * V, T);
        } else {
            ggml_tensor *o = b.alloc_result(GGML_TYPE_F32, H * V, T);
            b.ext(o, B200_EXT_MLSTM_SCAN, {part("mix.q", H * D), part("mix.k", H * D), part("mix.v", H * V), part("mix.i", H), part("mix.f", H), L.ib, L.fb, seq_info, L.state});
            o->op_params[2] = (int32_t)H; o->op_params[3] = (int32_t)D; o->op_params[4] = (int32_t)V;
            Builder::set_f(o, 5, lp.gate_cap); Builder::set_f(o, 6, 1.0f / sqrtf((float)D));
            ggml_tensor *on = norm(nullptr, b.reshape(o, V, H * T), L.mnorm, B200_NORM_RMS, H);   // per head, then the weight over all heads
            og = sigmoid_mul(b.reshape(on, H * V, T), part("mix.g", H * V));
        }
        ggml_tensor *y = b.mul_mat(L.wo, og);
        const bool mlp = lp.mlp != B200_MLP_NONE;
        ggml_tensor *x1 = norm(mlp ? nullptr : slice(il + 1), y, L.norm1b, B200_NORM_LAYER, 1, part("rg1", W), L.rg1b, x);
        if (mlp) {
            ggml_tensor *h2 = norm(nullptr, x1, L.norm2, B200_NORM_LAYER);
            ggml_tensor *P2 = b.mul_mat(L.proj2, h2);
            ggml_tensor *up = b.view_2d(P2, lp.ff, T, P2->nb[1], 0);
            ggml_tensor *a = b.ext(b.alloc_result(GGML_TYPE_F32, lp.ff, T), B200_EXT_POLYNORM, {up, L.act});
            Builder::set_f(a, 3, eps);
            ggml_tensor *y2 = b.mul_mat(L.down, a);
            x1 = norm(slice(il + 1), y2, L.norm2b, B200_NORM_LAYER, 1, b.view_2d(P2, W, T, P2->nb[1], (size_t)lp.ff * 4), L.rg2b, x1);
        }
        // what the next layer (or the output) reads: the learned mix of the embedding output and all results so far
        ggml_tensor *upto = b.view_3d(stack, W, T, il + 2, stack->nb[1], stack->nb[2], 0);
        upto->src[0] = x1;  // the newest slice is this layer's result: keep the dependency in the graph
        x = b.ext(b.alloc_result(GGML_TYPE_F32, W, T), B200_EXT_WEIGHTED_SUM, {upto, L.dwa});
    }
    b.bump = &m->regions[R_TAIL];
    ggml_tensor *out = x;
    if (bs.n_outputs > 0) {
        if (bs.n_outputs < T) out = b.get_rows(out, input_view(m->inp_out_ids, bs.n_outputs));
        out = b.mul_mat(g->head, norm(nullptr, out, g->final_norm, B200_NORM_LAYER));
    }
    b.expand(out);
    for (Bump &r : m->regions) LL_REQUIRE(m->measuring || r.off <= r.size, B200_ERR_NOMEM, "b200_llama_decode_batch: compute buffer too small for this batch");
    LL_REQUIRE(!b.oom, B200_ERR_NOMEM, "b200_llama_decode_batch: compute buffer too small for this batch");
    m->logits_t = bs.n_outputs > 0 ? out : nullptr;
    m->graph_nodes.swap(b.nodes);
    memset(&m->graph, 0, sizeof(m->graph));
    m->graph.size = m->graph.n_nodes = (int)m->graph_nodes.size();
    m->graph.nodes = m->graph_nodes.data();
    return B200_OK;
}

const Arch k_genesun = {"genesun", gs_place_tensor, gs_finalize, nullptr, gs_build, nullptr};

}  // namespace

const Arch *b200::host::genesun_arch() { return &k_genesun; }
