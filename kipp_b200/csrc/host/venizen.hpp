// Venizen: a decoder whose layers come in two kinds, listed one by one in its config.json.
//
//   parallel        an attention mixer and a retention mixer side by side on the same input,
//                   summed with a scale each.  The attention has grouped key/value heads, value
//                   heads of a size of their own, per-head q/k RMSNorm before a (partial) rotation,
//                   a matrix that mixes the heads' scores before the softmax, and a sliding window
//                   that keeps the first tokens of the sequence.
//   general_delta   the generalized delta rule (recurrent_parts.hpp).
//
// A layer's feed-forward is dense with a PolyNorm activation, or absent.  A span of layers
// ('loop': start, stop, times) runs several times in a row with the same weights; each pass has
// its own cache and state, and before each pass but the first the embedding output is added to
// the residual stream.  Then the model's norm and the output head.
//
// config.json keys: architecture, vocab, width, norm.eps, layers[i].{type, mixer, mlp}, loop.
// Tensor names: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
#pragma once
#include "model.hpp"

namespace kipp {
namespace venizen {

inline const Json& need(const Json& o, const char* key, const std::string& where) {
    const Json* v = o.is_object() ? o.find(key) : nullptr;
    if (!v || v->is_null()) fail(KIPP_E_CONFIG, "config.json lacks '" + where + key + "'");
    return *v;
}
inline long long need_int(const Json& o, const char* key, const std::string& where, long long least = 1) {
    const Json& v = need(o, key, where);
    if (v.is_bool() || !v.is_number() || (v.kind() == Json::Real && std::floor(v.as_double()) != v.as_double()))
        fail(KIPP_E_CONFIG, "config key '" + where + key + "' must be an integer, got " + v.dump());
    if (v.as_int() < least) fail(KIPP_E_CONFIG, format("config key '%s%s' must be at least %lld", where.c_str(), key, least));
    return v.as_int();
}
inline double need_number(const Json& o, const char* key, const std::string& where) {
    const Json& v = need(o, key, where);
    if (v.is_bool() || !v.is_number()) fail(KIPP_E_CONFIG, "config key '" + where + key + "' must be a number, got " + v.dump());
    return v.as_double();
}

// rot: {base, dims}; absent or dims 0 = no rotation
inline Json rotation(const Json& mixer, long long dim, const std::string& where) {
    Json out = Json::object();
    const Json* rot = mixer.find("rot");
    if (!rot || rot->is_null()) {
        out.set("dims", 0LL);
        out.set("base", 10000.0);
        return out;
    }
    const long long dims = need_int(*rot, "dims", where + "rot.", 0);
    if (dims % 2 || dims > dim) fail(KIPP_E_CONFIG, "config key '" + where + "rot.dims' must be even and at most the head's dim");
    const double base = dims > 0 ? need_number(*rot, "base", where + "rot.") : 10000.0;
    if (!(base > 0)) fail(KIPP_E_CONFIG, "config key '" + where + "rot.base' must be positive");
    out.set("dims", dims);
    out.set("base", base);
    return out;
}

// The keys after checks; every size and constant a model of this design can choose is kept.
inline Json normalize(const Json& c) {
    if (!c.is_object()) fail(KIPP_E_CONFIG, "config.json must hold a JSON object");
    Json out = Json::object();
    out.set("architecture", architecture_of(c));
    out.set("vocab", need_int(c, "vocab", ""));
    out.set("width", need_int(c, "width", ""));
    const double eps = need_number(need(c, "norm", ""), "eps", "norm.");
    if (!(eps > 0)) fail(KIPP_E_CONFIG, "norm.eps must be positive");
    Json norm = Json::object();
    norm.set("eps", eps);
    out.set("norm", std::move(norm));
    const Json& layers = need(c, "layers", "");
    if (!layers.is_array() || layers.size() == 0) fail(KIPP_E_CONFIG, "config key 'layers' must be a list of layers");
    Json ls = Json::array();
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& l = layers.at(i);
        const std::string where = format("layers[%zu].", i);
        const Json& type = need(l, "type", where);
        if (!type.is_string()) fail(KIPP_E_CONFIG, "config key '" + where + "type' must be a string");
        const Json& mx = need(l, "mixer", where);
        Json layer = Json::object(), mixer = Json::object();
        layer.set("type", type.as_string());
        if (type.as_string() == "parallel") {
            const Json& left = need(mx, "left", where + "mixer.");
            const Json& right = need(mx, "right", where + "mixer.");
            const std::string wl = where + "mixer.left.", wr = where + "mixer.right.";
            Json a = Json::object();
            const long long heads = need_int(left, "heads", wl), kv = need_int(left, "kv_heads", wl);
            const long long dim = need_int(left, "dim", wl);
            if (heads % kv) fail(KIPP_E_CONFIG, "config key '" + wl + "heads' must be a multiple of kv_heads");
            if (dim % 2) fail(KIPP_E_CONFIG, "config key '" + wl + "dim' must be even");
            a.set("heads", heads);
            a.set("kv_heads", kv);
            a.set("dim", dim);
            a.set("vdim", left.has("vdim") && !left.get("vdim").is_null() ? need_int(left, "vdim", wl) : dim);
            a.set("scale", need_number(left, "scale", wl));
            a.set("rot", rotation(left, dim, wl));
            Json mask = Json::object();
            if (const Json* m = left.find("mask"); m && !m->is_null()) {
                mask.set("size", need_int(*m, "size", wl + "mask."));
                mask.set("keep_first", m->has("keep_first") ? need_int(*m, "keep_first", wl + "mask.", 0) : 0LL);
            } else {                                   // no mask: every earlier token is seen
                mask.set("size", 0LL);
                mask.set("keep_first", 0LL);
            }
            a.set("mask", std::move(mask));
            Json r = Json::object();
            const long long rheads = need_int(right, "heads", wr), rdim = need_int(right, "dim", wr);
            if (rdim % 2) fail(KIPP_E_CONFIG, "config key '" + wr + "dim' must be even");
            r.set("heads", rheads);
            r.set("dim", rdim);
            r.set("vdim", right.has("vdim") && !right.get("vdim").is_null() ? need_int(right, "vdim", wr) : rdim);
            r.set("rot", rotation(right, rdim, wr));
            const Json& decay = need(right, "decay", wr);
            if (!decay.is_array() || (long long)decay.size() != rheads)
                fail(KIPP_E_CONFIG, "config key '" + wr + "decay' must list one decay per head");
            Json d = Json::array();
            for (auto& v : decay.items()) {
                if (!v.is_number()) fail(KIPP_E_CONFIG, "config key '" + wr + "decay' must hold numbers");
                d.push(v.as_double());
            }
            r.set("decay", std::move(d));
            mixer.set("left", std::move(a));
            mixer.set("right", std::move(r));
            mixer.set("left_scale", need_number(mx, "left_scale", where + "mixer."));
            mixer.set("right_scale", need_number(mx, "right_scale", where + "mixer."));
        } else if (type.as_string() == "general_delta") {
            mixer.set("heads", need_int(mx, "heads", where + "mixer."));
            mixer.set("dim", need_int(mx, "dim", where + "mixer."));
            // the width of the decay's bottleneck is the shape of its tensors unless a key gives it
            // (the random-weights writer needs it)
            if (const Json* r = mx.find("decay_rank"); r && !r->is_null())
                mixer.set("decay_rank", need_int(mx, "decay_rank", where + "mixer."));
        } else {
            fail(KIPP_E_CONFIG, "unknown layer type '" + type.as_string() + "' (parallel, general_delta)");
        }
        layer.set("mixer", std::move(mixer));
        const Json* mlp = l.find("mlp");
        if (mlp && !mlp->is_null()) {
            const std::string kind = mlp->get_string("kind", "dense");
            if (kind != "dense") fail(KIPP_E_CONFIG, "feed-forward kind '" + kind + "' is not supported (dense)");
            Json f = Json::object();
            f.set("kind", kind);
            f.set("ff", need_int(*mlp, "ff", where + "mlp."));
            layer.set("mlp", std::move(f));
        } else {
            layer.set("mlp", nullptr);
        }
        ls.push(std::move(layer));
    }
    const long long n_layers = (long long)ls.size();
    out.set("layers", std::move(ls));
    Json loop = Json::object();
    long long start = 0, stop = 0, times = 1;
    if (const Json* lp = c.find("loop"); lp && !lp->is_null()) {
        start = need_int(*lp, "start", "loop.", 0);
        stop = need_int(*lp, "stop", "loop.", 0);
        times = need_int(*lp, "times", "loop.", 1);
        if (start > stop || stop > n_layers) fail(KIPP_E_CONFIG, "loop: start <= stop <= number of layers is needed");
    }
    loop.set("start", start);
    loop.set("stop", stop);
    loop.set("times", times);
    out.set("loop", std::move(loop));
    return out;
}

inline Json rmsnorm_part(long long size, double eps, const char* weight_name) {
    Json j = Json::object();
    j.set("kind", "rmsnorm");
    j.set("size", size);
    j.set("eps", eps);
    j.set("weight_name", weight_name);
    return j;
}
inline Json rotary_part(const Json& rot, long long dim) {
    Json j = Json::object();
    if (rot.get("dims").as_int() == 0) {
        j.set("kind", "no_position");
        return j;
    }
    j.set("kind", "rotary");
    j.set("head_dim", dim);
    j.set("rotary_dim", rot.get("dims").as_int());
    j.set("theta", rot.get("base").as_double());
    j.set("exact_exponent", true);          // f_i is the real number base^(-2i/dims), rounded once
    return j;
}
inline Json names_of(std::initializer_list<std::pair<const char*, const char*>> pairs) {
    Json j = Json::object();
    for (auto& p : pairs) j.set(p.first, p.second);
    return j;
}

inline Json plan(const Json& c) {
    const long long width = c.get("width").as_int(), vocab = c.get("vocab").as_int();
    const double eps = c.get("norm").get("eps").as_double();
    Json p = Json::object();
    p.set("hidden_size", width);
    p.set("vocab_size", vocab);
    p.set("max_positions", 0LL);
    p.set("config", c);
    Json emb = Json::object();
    emb.set("kind", "token_embedding");
    emb.set("vocab_size", vocab);
    emb.set("hidden_size", width);
    emb.set("weight_name", "embed");
    Json stage = Json::object();
    stage.set("prefix", "");
    stage.set("part", std::move(emb));
    Json stages = Json::array();
    stages.push(std::move(stage));
    p.set("embedding", std::move(stages));

    Json blocks = Json::array();
    const Json& layers = c.get("layers");
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& l = layers.at(i);
        const Json& mx = l.get("mixer");
        Json mixer = Json::object();
        if (l.get("type").as_string() == "parallel") {
            const Json& a = mx.get("left");
            const Json& r = mx.get("right");
            Json attn = Json::object();
            attn.set("kind", "attention");
            attn.set("hidden_size", width);
            attn.set("num_heads", a.get("heads").as_int());
            attn.set("num_kv_heads", a.get("kv_heads").as_int());
            attn.set("head_dim", a.get("dim").as_int());
            attn.set("value_dim", a.get("vdim").as_int());
            attn.set("position", rotary_part(a.get("rot"), a.get("dim").as_int()));
            attn.set("qk_norm_eps", eps);
            attn.set("scale", a.get("scale").as_double());
            attn.set("window", a.get("mask").get("size").as_int());
            attn.set("keep_first", a.get("mask").get("keep_first").as_int());
            attn.set("head_mix", true);
            attn.set("output_scale", mx.get("left_scale").as_double());
            attn.set("names", names_of({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"o", "o"}, {"q_norm", "q.norm"},
                                        {"k_norm", "k.norm"}, {"head_mix", "talk"}}));
            Json ret = Json::object();
            ret.set("kind", "retention");
            ret.set("hidden_size", width);
            ret.set("num_heads", r.get("heads").as_int());
            ret.set("head_dim", r.get("dim").as_int());
            ret.set("value_dim", r.get("vdim").as_int());
            ret.set("position", rotary_part(r.get("rot"), r.get("dim").as_int()));
            ret.set("decay", r.get("decay"));
            ret.set("eps", eps);
            ret.set("gate", "silu");
            ret.set("output_scale", mx.get("right_scale").as_double());
            Json branches = Json::array();
            Json bl = Json::object(), br = Json::object();
            bl.set("prefix", "left.");
            bl.set("part", std::move(attn));
            br.set("prefix", "right.");
            br.set("part", std::move(ret));
            branches.push(std::move(bl));
            branches.push(std::move(br));
            mixer.set("kind", "parallel");
            mixer.set("branches", std::move(branches));
        } else {
            mixer.set("kind", "delta_rule");
            mixer.set("hidden_size", width);
            mixer.set("num_heads", mx.get("heads").as_int());
            mixer.set("head_dim", mx.get("dim").as_int());
            mixer.set("decay_rank", mx.get_int("decay_rank", 0));
            mixer.set("eps", eps);
            mixer.set("gate", "sigmoid");
        }
        Json block = Json::object();
        block.set("kind", "pre_norm_block");
        Json names = Json::array();
        for (const char* n : {"", "mix.", "", "mlp."}) names.push(n);
        block.set("names", std::move(names));
        block.set("input_norm", rmsnorm_part(width, eps, "norm1"));
        block.set("mixer", std::move(mixer));
        if (!l.get("mlp").is_null()) {
            Json ffn = Json::object();
            ffn.set("kind", "polynorm_mlp");
            ffn.set("hidden_size", width);
            ffn.set("intermediate_size", l.get("mlp").get("ff").as_int());
            ffn.set("eps", eps);
            block.set("post_norm", rmsnorm_part(width, eps, "norm2"));
            block.set("ffn", std::move(ffn));
        } else {
            block.set("post_norm", nullptr);
            block.set("ffn", nullptr);
        }
        Json layer = Json::object();
        layer.set("prefix", format("l%zu.", i));
        layer.set("part", std::move(block));
        blocks.push(std::move(layer));
    }
    p.set("layers", std::move(blocks));

    // the order: layers before the span, the span `times` times (each pass with caches and states
    // of its own, the embedding output added before every pass but the first), the rest
    Json order = Json::array();
    const long long n = (long long)layers.size();
    const long long start = c.get("loop").get("start").as_int(), stop = c.get("loop").get("stop").as_int();
    const long long times = c.get("loop").get("times").as_int();
    long long cache = 0;
    auto push = [&](long long layer, bool adds) {
        Json run = Json::object();
        run.set("layer", layer);
        run.set("cache", cache++);
        run.set("writes_cache", true);
        run.set("adds_embedding", adds);
        order.push(std::move(run));
    };
    for (long long i = 0; i < start; ++i) push(i, false);
    for (long long t = 0; t < times; ++t)
        for (long long i = start; i < stop; ++i) push(i, t > 0 && i == start);
    for (long long i = stop; i < n; ++i) push(i, false);
    p.set("order", std::move(order));

    Json fn = Json::object();
    fn.set("prefix", "");
    fn.set("part", rmsnorm_part(width, eps, "final.norm"));
    p.set("final_norm", std::move(fn));
    Json head = Json::object();
    head.set("kind", "output_head");
    head.set("vocab_size", vocab);
    head.set("hidden_size", width);
    head.set("tied_to", nullptr);
    head.set("weight_name", "head");
    Json hd = Json::object();
    hd.set("prefix", "");
    hd.set("part", std::move(head));
    p.set("head", std::move(hd));
    return p;
}

}  // namespace venizen

inline void register_venizen() {
    Registry::get().add_architecture("Venizen", Architecture{venizen::normalize, venizen::plan});
}

}  // namespace kipp
