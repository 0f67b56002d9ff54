// Part kinds beyond plain grouped-query attention: softmax attention with a sink and a learned
// bias by distance, the gated delta rule, and a pre-norm block that runs two mixers side by side.
// Every size and constant is a parameter; no kind knows which model it is in.
#include <cmath>

#include "kernels.h"
#include "ops.hpp"
#include "parts.hpp"

namespace imp {

namespace {

int64_t need_int(const Json& p, const char* key, const char* part) {
    const Json* v = p.find(key);
    if (!v || !v->is_number()) fail(IMP_ERROR_INVALID_MODEL, std::string(part) + ": parameter '" + key + "' is missing");
    return v->as_int();
}
double need_double(const Json& p, const char* key, const char* part) {
    const Json* v = p.find(key);
    if (!v || !v->is_number()) fail(IMP_ERROR_INVALID_MODEL, std::string(part) + ": parameter '" + key + "' is missing");
    return v->as_double();
}

// A small tensor of the model as 32-bit values on the host.
std::vector<float> to_host_f32(Runtime& rt, WeightStore& store, const Tensor& t) {
    Tensor f = to_float32(rt, store, t);
    std::vector<float> out((size_t)numel(t));
    IMP_CUDA(cudaMemcpyAsync(out.data(), f.data, out.size() * 4, cudaMemcpyDeviceToHost, rt.stream));
    IMP_CUDA(cudaStreamSynchronize(rt.stream));
    store.release(f.data);
    return out;
}

// -------------------------------------------------------------------- attention with sink and bias
// Softmax attention over the paged cache without a rotation and without a value projection:
//   q = Wq x + bq, k = Wk x + bk; the value of a token is k (as projected);
//   q and k are RMS-normalised over the whole projection (all heads at once) with plain weights;
//   q is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1) at position p;
//   score(i, j) = scale * q_i . k_j + rel[bucket(i - j), head]; the softmax denominator also holds
//   exp(sink[head]); out = Wo attn + bo.
// bucket(n) = n below half the table, then logarithmic up to `bias_max_distance`, then the last row.
// The table by bucket is expanded at load into a table by distance, [heads, bias_max_distance + 1].
//
// params: hidden_size, num_heads, num_kv_heads, head_dim, scale, norm_eps, q_temp_coef, q_temp_every
//         (0 = none), bias_max_distance, bias_buckets (0 or absent: the rows of the checkpoint's table),
//         window (0 = all).
struct SinkBiasAttention : Mixer {
    AttentionGeometry g;
    Tensor w_qk, w_o;
    Tensor b_q, b_k, b_o, n_q, n_k, sink, bias_by_distance;   // float32
    Tensor sink_l2, bias_l2, bias_pad_l2;                      // the last two times log2(e), for kernels that use 2^x; and padded
    float eps, temp_coef;
    int temp_every, n_dist;
    bool bias_deferred = false;
    const float* defer_out_bias() override {
        bias_deferred = true;
        return (const float*)b_o.data;
    }

    static TensorSpecs specs(const Json& p) {
        const char* me = "sink_bias_attention";
        const int64_t d = need_int(p, "hidden_size", me), hq = need_int(p, "num_heads", me), hkv = need_int(p, "num_kv_heads", me),
                      dh = need_int(p, "head_dim", me), nb = p.get_int("bias_buckets", 0);   // 0: as many rows as the checkpoint's table has
        TensorSpecs s;
        s.emplace_back("q_proj", TensorSpec{{hq * dh, d}});
        s.emplace_back("q_bias", TensorSpec{{hq * dh}, "vector", "normal"});
        s.emplace_back("k_proj", TensorSpec{{hkv * dh, d}});
        s.emplace_back("k_bias", TensorSpec{{hkv * dh}, "vector", "normal"});
        s.emplace_back("q_norm", TensorSpec{{hq * dh}, "norm", "one_plus_normal"});
        s.emplace_back("k_norm", TensorSpec{{hkv * dh}, "norm", "one_plus_normal"});
        s.emplace_back("rel_bias", TensorSpec{{nb > 0 ? nb : -1, hq}, "vector", "normal"});
        s.emplace_back("sink", TensorSpec{{hq}, "vector", "normal"});
        s.emplace_back("o_proj", TensorSpec{{d, hq * dh}});
        s.emplace_back("o_bias", TensorSpec{{d}, "vector", "normal"});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        return CacheSpec::paged((int)need_int(p, "num_kv_heads", "sink_bias_attention"), (int)need_int(p, "head_dim", "sink_bias_attention"),
                                (int)p.get_int("window", 0));
    }
    // Row of the bias table for distance n >= 0.
    static int bucket(int64_t n, int64_t n_buckets, int64_t max_distance) {
        const int64_t half = n_buckets / 2;
        if (n < half) return (int)n;
        const double r = std::log((double)n / (double)half) / std::log((double)max_distance / (double)half) * (double)(n_buckets - half);
        return (int)std::min<int64_t>(n_buckets - 1, half + (int64_t)std::floor(r));
    }

    explicit SinkBiasAttention(BuildArgs& a) {
        const char* me = "sink_bias_attention";
        const Json& p = a.params;
        g.hq = (int)need_int(p, "num_heads", me);
        g.hkv = (int)need_int(p, "num_kv_heads", me);
        g.dh = (int)need_int(p, "head_dim", me);
        g.window = (int)p.get_int("window", 0);
        g.scale = (float)need_double(p, "scale", me);
        if (g.hkv <= 0 || g.hq % g.hkv)
            fail(IMP_ERROR_INVALID_MODEL, std::to_string(g.hq) + " query heads are not a multiple of " + std::to_string(g.hkv) + " kv heads");
        if (g.dh <= 0 || g.dh > 256) fail(IMP_ERROR_INVALID_MODEL, "head_dim " + std::to_string(g.dh) + " must lie in (0, 256]");
        eps = (float)p.get_double("norm_eps", 1e-6);
        temp_coef = (float)p.get_double("q_temp_coef", 0.0);
        temp_every = (int)p.get_int("q_temp_every", 0);
        const int64_t nb = a.tensor("rel_bias").shape[0], dmax = need_int(p, "bias_max_distance", me);
        if (nb < 2 || dmax <= nb / 2)
            fail(IMP_ERROR_INVALID_MODEL, "bias_max_distance " + std::to_string(dmax) + " must exceed half of the " + std::to_string(nb) + " buckets");
        Runtime& rt = *a.rt;
        w_qk = cat_rows(rt, *a.store, {a.tensor("q_proj"), a.tensor("k_proj")});
        w_o = a.tensor("o_proj");
        b_q = to_float32(rt, *a.store, a.tensor("q_bias"));
        b_k = to_float32(rt, *a.store, a.tensor("k_bias"));
        b_o = to_float32(rt, *a.store, a.tensor("o_bias"));
        n_q = to_float32(rt, *a.store, a.tensor("q_norm"));
        n_k = to_float32(rt, *a.store, a.tensor("k_norm"));
        sink = to_float32(rt, *a.store, a.tensor("sink"));
        // the table by bucket [buckets, heads] becomes a table by distance [heads, dmax + 1]: every distance from dmax on
        // reads the last bucket
        const std::vector<float> rel = to_host_f32(rt, *a.store, a.tensor("rel_bias"));
        n_dist = (int)dmax + 1;
        std::vector<float> tab((size_t)g.hq * (size_t)n_dist);
        for (int h = 0; h < g.hq; ++h)
            for (int n = 0; n < n_dist; ++n) tab[(size_t)h * n_dist + n] = rel[(size_t)bucket(n, nb, dmax) * g.hq + h];
        bias_by_distance = a.store->alloc(F32, {g.hq, n_dist});
        IMP_CUDA(cudaMemcpyAsync(bias_by_distance.data, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        const double log2e = 1.4426950408889634;
        std::vector<float> sk = to_host_f32(rt, *a.store, sink);
        for (float& v : tab) v = (float)((double)v * log2e);
        for (float& v : sk) v = (float)((double)v * log2e);
        bias_l2 = a.store->alloc(F32, {g.hq, n_dist});
        sink_l2 = a.store->alloc(F32, {g.hq});
        IMP_CUDA(cudaMemcpyAsync(bias_l2.data, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        IMP_CUDA(cudaMemcpyAsync(sink_l2.data, sk.data(), sk.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        // the padded layout of the tensor-memory kernel: zeros in front, the last entry repeated behind
        const int pad = ATTENTION_BIAS_PAD, row = n_dist + 2 * pad;
        std::vector<float> padded((size_t)g.hq * (size_t)row, 0.f);
        for (int h = 0; h < g.hq; ++h)
            for (int n = 0; n < n_dist + pad; ++n) padded[(size_t)h * row + pad + n] = tab[(size_t)h * n_dist + std::min(n, n_dist - 1)];
        bias_pad_l2 = a.store->alloc(F32, {g.hq, row});
        IMP_CUDA(cudaMemcpyAsync(bias_pad_l2.data, padded.data(), padded.size() * 4, cudaMemcpyHostToDevice, rt.stream));
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        for (const char* n : {"q_proj", "k_proj", "q_bias", "k_bias", "o_bias", "q_norm", "k_norm", "sink", "rel_bias"}) a.drop(n);
    }

    std::vector<TilingSpec> tilings() const override { return attention_tilings(); }

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || !cache->paged()) fail(IMP_ERROR_INTERNAL, "sink_bias_attention runs against a paged cache");
        const int64_t T = rows(x);
        const int64_t qd = (int64_t)g.hq * g.dh, kd = (int64_t)g.hkv * g.dh;
        const ImpCacheView& cv = cache->view;
        Tensor qk = rt.empty(T, qd + kd);
        linear(rt, qk, x, w_qk);
        ++rt.launches;
        check_launch(imp_proj_norm_kv_write(qk.data, qk.stride0, (int)T, g.hq, g.hkv, g.dh, (const float*)b_q.data, (const float*)b_k.data,
                                            (const float*)n_q.data, (const float*)n_k.data, eps, temp_coef, temp_every, st.view.positions,
                                            st.view.seq_of_token, cv.block_table, cv.bt_stride, st.B(), cv.writes ? cv.k_pages : nullptr,
                                            cv.writes ? cv.v_pages : nullptr, cv.page_size, cv.num_pages, rt.dtype, rt.status, rt.stream),
                     "proj_norm_kv_write");
        Tensor attn = rt.empty(T, qd);
        AttentionExtras ex;
        ex.bias = (const float*)bias_by_distance.data;
        ex.n_dist = n_dist;
        ex.sink = (const float*)sink.data;
        ex.bias_l2 = (const float*)bias_l2.data;
        ex.sink_l2 = (const float*)sink_l2.data;
        ex.bias_pad_l2 = (const float*)bias_pad_l2.data;
        ex.pad = ATTENTION_BIAS_PAD;
        paged_attention(st, attn, col_slice(qk, 0, qd), g, *cache, tiling_ids, &ex);
        Tensor out = rt.empty(T, rows(w_o));
        linear(rt, out, attn, w_o);
        if (!bias_deferred) {
            ++rt.launches;
            check_launch(imp_add_bias(out.data, out.stride0, (int)T, (int)cols(out), (const float*)b_o.data, out.dtype, rt.stream), "add_bias");
        }
        return Branch::of(out);
    }
};

// ------------------------------------------------------------------------------ gated delta rule
// A recurrent mixer with a matrix state per head (see csrc/delta_rule.cu for the recurrence):
//   q, k [G heads of D], v [H heads of Dv] = silu(conv(W x)) with a causal convolution of `conv_taps` taps per channel;
//   q, k unit vectors per head, q times D^(-1/2); beta = sigmoid(Wb x); decay = exp(-exp(A_log) softplus(Wa x + dt_bias));
//   o = recurrence; y = o / rms(o) * w_norm * silu(Wg x) per head; out = Wo y.
// One product makes q, k, v, the gate, beta's and the decay's inputs; its rows are padded to a multiple of 8.
// State per request: S (H heads of D x Dv, in the scan kernel's layout) and the last conv_taps - 1 inputs of the
// convolution, both float32.
//
// params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv_taps, norm_eps.
struct GatedDeltaRule : Mixer {
    int H, G, D, Dv, taps;
    float eps;
    Tensor w_in, w_o, conv_w, a_log, dt_bias, out_norm;   // the last four float32

    struct Sizes {
        int64_t d, H, G, D, Dv, taps;
        int64_t channels() const { return 2 * G * D + H * Dv; }
    };
    static Sizes sizes(const Json& p) {
        const char* me = "gated_delta_rule";
        Sizes s{need_int(p, "hidden_size", me), need_int(p, "num_heads", me), need_int(p, "num_kv_heads", me), need_int(p, "key_dim", me),
                need_int(p, "value_dim", me), need_int(p, "conv_taps", me)};
        if (s.G <= 0 || s.H <= 0 || s.H % s.G) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": " + std::to_string(s.H) + " heads over " + std::to_string(s.G) + " key heads");
        if (s.D <= 0 || s.D > 256 || s.Dv <= 0) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": key_dim must lie in (0, 256] and value_dim be positive");
        if (s.taps < 1 || s.taps > 64) fail(IMP_ERROR_INVALID_MODEL, std::string(me) + ": conv_taps must lie in [1, 64]");
        return s;
    }
    static TensorSpecs specs(const Json& p) {
        const Sizes z = sizes(p);
        TensorSpecs s;
        s.emplace_back("q_proj", TensorSpec{{z.G * z.D, z.d}});
        s.emplace_back("q_conv", TensorSpec{{z.G * z.D, z.taps}, "vector", "normal"});
        s.emplace_back("k_proj", TensorSpec{{z.G * z.D, z.d}});
        s.emplace_back("k_conv", TensorSpec{{z.G * z.D, z.taps}, "vector", "normal"});
        s.emplace_back("v_proj", TensorSpec{{z.H * z.Dv, z.d}});
        s.emplace_back("v_conv", TensorSpec{{z.H * z.Dv, z.taps}, "vector", "normal"});
        s.emplace_back("beta_proj", TensorSpec{{z.H, z.d}});
        s.emplace_back("a_log", TensorSpec{{z.H}, "vector", "normal"});
        s.emplace_back("out_norm", TensorSpec{{z.Dv}, "norm", "one_plus_normal"});
        s.emplace_back("a_proj", TensorSpec{{z.H, z.d}});
        s.emplace_back("dt_bias", TensorSpec{{z.H}, "vector", "normal"});
        s.emplace_back("gate_proj", TensorSpec{{z.H * z.Dv, z.d}});
        s.emplace_back("o_proj", TensorSpec{{z.d, z.H * z.Dv}});
        return s;
    }
    static CacheSpec cache(const Json& p) {
        const Sizes z = sizes(p);
        CacheSpec s;
        s.kind = CacheSpec::State;
        // S in the scan kernel's own layout (whole lanes and column blocks; see csrc/delta_rule.cu)
        s.states.push_back(StateTensorSpec{"S", {imp_gdr_state_floats((int)z.H, (int)z.D, (int)z.Dv)}, F32});
        s.states.push_back(StateTensorSpec{"conv", {std::max<int64_t>(z.taps - 1, 1), z.channels()}, F32});
        return s;
    }

    explicit GatedDeltaRule(BuildArgs& a) {
        const Sizes z = sizes(a.params);
        H = (int)z.H, G = (int)z.G, D = (int)z.D, Dv = (int)z.Dv, taps = (int)z.taps;
        eps = (float)a.params.get_double("norm_eps", 1e-6);
        Runtime& rt = *a.rt;
        std::vector<Tensor> in = {a.tensor("q_proj"), a.tensor("k_proj"), a.tensor("v_proj"), a.tensor("gate_proj"), a.tensor("beta_proj"),
                                  a.tensor("a_proj")};
        const int64_t n = z.channels() + z.H * z.Dv + 2 * z.H, pad = (8 - n % 8) % 8;
        Tensor zeros{};
        if (pad) {
            zeros = a.store->alloc(in[0].dtype, {pad, z.d});
            IMP_CUDA(cudaMemsetAsync(zeros.data, 0, (size_t)numel(zeros) * elem_size(zeros.dtype), rt.stream));
            in.push_back(zeros);
        }
        w_in = cat_rows(rt, *a.store, in);
        w_o = a.tensor("o_proj");
        Tensor cw = cat_rows(rt, *a.store, {a.tensor("q_conv"), a.tensor("k_conv"), a.tensor("v_conv")});
        conv_w = to_float32(rt, *a.store, cw);
        a_log = to_float32(rt, *a.store, a.tensor("a_log"));
        dt_bias = to_float32(rt, *a.store, a.tensor("dt_bias"));
        out_norm = to_float32(rt, *a.store, a.tensor("out_norm"));
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        a.store->release(cw.data);
        if (pad) a.store->release(zeros.data);
        for (const char* n2 : {"q_proj", "k_proj", "v_proj", "gate_proj", "beta_proj", "a_proj", "q_conv", "k_conv", "v_conv", "a_log", "dt_bias",
                               "out_norm"})
            a.drop(n2);
    }

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || cache->view.kind != 2 || cache->view.n_states < 2) fail(IMP_ERROR_INTERNAL, "gated_delta_rule runs against a state cache");
        const int64_t T = rows(x);
        const int C = 2 * G * D + H * Dv;
        Tensor proj = rt.empty(T, rows(w_in));
        linear(rt, proj, x, w_in);
        float* qn = rt.arena->take<float>((size_t)T * G * D);
        float* kn = rt.arena->take<float>((size_t)T * G * D);
        float* vc = rt.arena->take<float>((size_t)T * H * Dv);
        float* beta = rt.arena->take<float>((size_t)T * H);
        float* decay = rt.arena->take<float>((size_t)T * H);
        float* o = rt.arena->take<float>((size_t)T * H * Dv);
        float* S = (float*)cache->view.states[0].data;
        float* conv_state = (float*)cache->view.states[1].data;
        // a step of single tokens: the convolution's state is rewritten by the kernel that reads it
        const bool single = st.decode_only();
        rt.launches += single ? 3 : 4;
        check_launch(imp_gdr_prepare(proj.data, proj.stride0, (const float*)conv_w.data, taps, conv_state, st.view.seq_of_token, st.view.q_start,
                                     st.view.state_slots, (int)T, st.B(), G, D, H, Dv, (const float*)a_log.data, (const float*)dt_bias.data, qn,
                                     kn, vc, beta, decay, single ? 1 : 0, rt.dtype, rt.status, rt.stream),
                     "gdr_prepare");
        if (!single)
            check_launch(imp_gdr_conv_state(proj.data, proj.stride0, conv_state, taps, C, st.view.q_start, st.view.state_slots, st.B(), rt.dtype,
                                            rt.stream),
                         "gdr_conv_state");
        check_launch(imp_gdr_scan(qn, kn, vc, beta, decay, S, o, st.view.q_start, st.view.state_slots, st.B(), G, D, H, Dv, rt.stream), "gdr_scan");
        Tensor y = rt.empty(T, (int64_t)H * Dv);
        const Tensor gate = col_slice(proj, C, (int64_t)H * Dv);
        check_launch(imp_gdr_output(y.data, o, gate.data, gate.stride0, (const float*)out_norm.data, eps, (int)T, H, Dv, rt.dtype, rt.stream),
                     "gdr_output");
        Tensor out = rt.empty(T, rows(w_o));
        linear(rt, out, y, w_o);
        return Branch::of(out);
    }
};

// --------------------------------------------------------------------------- two mixers side by side
// h += left_scale * left(norm1(h)) + right_scale * right(norm1(h)); then, if the layer has a feed-forward,
// h += ffn(norm2(h)).  Both mixers read the same normalised input and each owns a cache of its own.
// Slots: mixer_norm, left, right, and with has_ffn (default true) ffn_norm, feed_forward.
// params: left_scale, right_scale, has_ffn.
struct ParallelPreNormBlock : Block {
    Mixer *left, *right;
    FeedForward* ffn = nullptr;
    Norm *norm1, *norm2 = nullptr;
    float ls, rs;
    const float* left_bias = nullptr;      // the left mixer's output bias, added (times left_scale) where the two outputs are summed
    explicit ParallelPreNormBlock(BuildArgs& a)
        : left(part_cast<Mixer>(a.part("left"), "a mixer")), right(part_cast<Mixer>(a.part("right"), "a mixer")),
          norm1(part_cast<Norm>(a.part("mixer_norm"), "a norm")), ls((float)a.params.get_double("left_scale", 1.0)),
          rs((float)a.params.get_double("right_scale", 1.0)) {
        left_bias = left->defer_out_bias();
        if (a.params.get_bool("has_ffn", true)) {
            ffn = part_cast<FeedForward>(a.part("feed_forward"), "a feed-forward");
            norm2 = part_cast<Norm>(a.part("ffn_norm"), "a norm");
        }
    }
    static std::vector<Slot> slots(const Json& p) {
        std::vector<Slot> s = {{"mixer_norm", "norm"}, {"left", "mixer"}, {"right", "mixer"}};
        if (p.get_bool("has_ffn", true)) {
            s.push_back({"ffn_norm", "norm"});
            s.push_back({"feed_forward", "feed_forward"});
        }
        return s;
    }
    bool takes_split_sum() const override { return norm1->takes_split_sum(); }
    Mixer* mixer() const override { return left; }
    std::vector<Mixer*> mixers() const override { return {left, right}; }
    std::vector<Part*> parts() const override {
        std::vector<Part*> p = {norm1, left, right};
        if (ffn) {
            p.push_back(norm2);
            p.push_back(ffn);
        }
        return p;
    }
    bool graph_safe() const override {
        for (Part* p : parts())
            if (!p->graph_safe()) return false;
        return true;
    }
    Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache) fail(IMP_ERROR_INTERNAL, "parallel_prenorm needs the caches of its two mixers");
        Tensor x = norm1->add_norm(st, h, pending);
        Tensor a = summed(st, left->forward(st, x, cache[0].view.kind ? &cache[0] : nullptr));
        Tensor b = summed(st, right->forward(st, x, cache[1].view.kind ? &cache[1] : nullptr));
        Tensor sum = rt.empty(rows(a), cols(a));
        ++rt.launches;
        check_launch(imp_scaled_sum(sum.data, a.data, ls, b.data, rs, left_bias, ls, (int)rows(a), (int)cols(a), sum.dtype, rt.stream), "scaled_sum");
        stage(st, "mixer", sum);
        if (!ffn) return Branch::of(sum);
        x = norm2->add_norm(st, h, Branch::of(sum));
        ffn->defer_out = defer_pending;
        Branch f = ffn->forward(st, x);
        stage(st, "feed_forward", f);
        return f;
    }
};

template <typename T> PartClass class_of(TensorSpecs (*specs)(const Json&)) {
    PartClass c;
    if (specs) c.tensor_specs = specs;
    c.create = [](BuildArgs& a) -> Part* { return new T(a); };
    return c;
}

}  // namespace

void register_mixer_parts() {
    PartClass attn = class_of<SinkBiasAttention>(&SinkBiasAttention::specs);
    attn.cache_spec = &SinkBiasAttention::cache;
    register_part_class("mixer", "sink_bias_attention", attn, true);
    PartClass gdr = class_of<GatedDeltaRule>(&GatedDeltaRule::specs);
    gdr.cache_spec = &GatedDeltaRule::cache;
    register_part_class("mixer", "gated_delta_rule", gdr, true);
    PartClass block = class_of<ParallelPreNormBlock>(nullptr);
    block.part_slots = &ParallelPreNormBlock::slots;
    register_part_class("block", "parallel_prenorm", block, true);
}

}  // namespace imp
