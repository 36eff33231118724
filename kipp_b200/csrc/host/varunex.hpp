// Varunex: a decoder whose layers are listed one by one in its config.json, each with one of
// three mixers:
//
//   mlstm              the gated matrix memory (recurrent_parts.hpp, kind gated_memory);
//   latent_attention   attention over a cached latent with a shared rotated key part, a sink in
//                      the softmax's denominator and a gate per head (latent_parts.hpp);
//   attention          grouped-query attention with two score maps per head whose outputs are
//                      taken off each other (differential attention), biases on q, k and v, a
//                      rotation of the first dims of every map with stretched long wavelengths,
//                      and a sliding window (options of the attention mixer, parts.hpp).
//
// A layer is x <- x + mixer(n) + ff(n) with n = layer norm (weight and bias) of x: one norm, both
// sublayers read it (parallel_block).  The feed-forward is dense with the square of relu as its
// activation, or absent.  Then the model's layer norm and the output head.
//
// config.json keys: architecture, vocab, width, norm.eps, layers[i].{type, mixer, mlp}.
// Tensor names: embed, l<i>.norm1(.b), l<i>.mix.*, l<i>.mlp.{up,down}, final.norm(.b), head.
#pragma once
#include "venizen.hpp"

namespace kipp {
namespace varunex {

using venizen::need;
using venizen::need_int;
using venizen::need_number;

inline long long optional_int(const Json& o, const char* key, const std::string& where, long long fallback, long long least) {
    const Json* v = o.find(key);
    return v && !v->is_null() ? need_int(o, key, where, least) : fallback;
}

// rot: {base, dims, scaling: {factor, low, high, original}}; absent or dims 0 = no rotation
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
    if (const Json* sc = rot->find("scaling"); sc && !sc->is_null() && dims > 0) {
        const std::string ws = where + "rot.scaling.";
        Json s = Json::object();
        for (const char* key : {"factor", "low", "high", "original"}) s.set(key, need_number(*sc, key, ws));
        if (!(s.get("factor").as_double() > 0) || !(s.get("low").as_double() > 0) ||
            !(s.get("high").as_double() > s.get("low").as_double()) || !(s.get("original").as_double() > 0))
            fail(KIPP_E_CONFIG, "config key '" + ws + "*': factor, low and original must be positive and high above low");
        out.set("scaling", std::move(s));
    }
    return out;
}

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
        const std::string where = format("layers[%zu].", i), wm = where + "mixer.";
        const Json& type = need(l, "type", where);
        if (!type.is_string()) fail(KIPP_E_CONFIG, "config key '" + where + "type' must be a string");
        const Json& mx = need(l, "mixer", where);
        const std::string kind = type.as_string();
        Json layer = Json::object(), mixer = Json::object();
        layer.set("type", kind);
        if (kind == "mlstm") {
            const long long dim = need_int(mx, "dim", wm);
            mixer.set("heads", need_int(mx, "heads", wm));
            mixer.set("dim", dim);
            mixer.set("vdim", optional_int(mx, "vdim", wm, dim, 1));
            const double cap = need_number(mx, "gate_cap", wm);
            if (!(cap > 0)) fail(KIPP_E_CONFIG, "config key '" + wm + "gate_cap' must be positive");
            mixer.set("gate_cap", cap);
        } else if (kind == "latent_attention") {
            const long long dim = need_int(mx, "dim", wm), rot_dim = need_int(mx, "rot_dim", wm, 0);
            mixer.set("heads", need_int(mx, "heads", wm));
            mixer.set("dim", dim);
            mixer.set("rot_dim", rot_dim);
            mixer.set("vdim", optional_int(mx, "vdim", wm, dim, 1));
            mixer.set("kv_rank", need_int(mx, "kv_rank", wm));
            mixer.set("q_rank", need_int(mx, "q_rank", wm));
            mixer.set("scale", need_number(mx, "scale", wm));
            Json rot = rotation(mx, rot_dim, wm);
            if (rot.get("dims").as_int() != rot_dim)
                fail(KIPP_E_CONFIG, "config key '" + wm + "rot.dims' must equal rot_dim: the whole rotated part turns");
            mixer.set("rot", std::move(rot));
        } else if (kind == "attention") {
            const long long heads = need_int(mx, "heads", wm), kv = optional_int(mx, "kv_heads", wm, heads, 1);
            const long long dim = need_int(mx, "dim", wm);
            if (heads % kv) fail(KIPP_E_CONFIG, "config key '" + wm + "heads' must be a multiple of kv_heads");
            mixer.set("heads", heads);
            mixer.set("kv_heads", kv);
            mixer.set("dim", dim);
            mixer.set("vdim", optional_int(mx, "vdim", wm, dim, 1));
            mixer.set("scale", need_number(mx, "scale", wm));
            mixer.set("diff", need_number(mx, "diff", wm));
            mixer.set("rot", rotation(mx, dim, wm));
            Json mask = Json::object();
            const Json* m = mx.find("mask");
            mask.set("size", m && !m->is_null() ? need_int(*m, "size", wm + "mask.", 0) : 0LL);   // 0: every earlier token
            mixer.set("mask", std::move(mask));
        } else {
            fail(KIPP_E_CONFIG, "unknown layer type '" + kind + "' (mlstm, latent_attention, attention)");
        }
        layer.set("mixer", std::move(mixer));
        const Json* mlp = l.find("mlp");
        if (mlp && !mlp->is_null()) {
            const std::string fk = mlp->get_string("kind", "dense");
            if (fk != "dense") fail(KIPP_E_CONFIG, "feed-forward kind '" + fk + "' is not supported (dense)");
            Json f = Json::object();
            f.set("kind", fk);
            f.set("ff", need_int(*mlp, "ff", where + "mlp."));
            layer.set("mlp", std::move(f));
        } else {
            layer.set("mlp", nullptr);
        }
        ls.push(std::move(layer));
    }
    out.set("layers", std::move(ls));
    return out;
}

inline Json layernorm_part(long long size, double eps, const std::string& name) {
    Json j = Json::object();
    j.set("kind", "layernorm");
    j.set("size", size);
    j.set("eps", eps);
    j.set("weight_name", name);
    j.set("bias_name", name + ".b");
    return j;
}
inline Json rotary_part(const Json& rot, long long dim) {
    Json j = Json::object();
    if (rot.get("dims").as_int() == 0) {
        j.set("kind", "no_position");
        return j;
    }
    j.set("head_dim", dim);
    j.set("rotary_dim", rot.get("dims").as_int());
    j.set("theta", rot.get("base").as_double());
    if (const Json* sc = rot.find("scaling")) {
        j.set("kind", "stretched_rotary");
        for (const char* key : {"factor", "low", "high", "original"}) j.set(key, sc->get(key).as_double());
    } else {
        j.set("kind", "rotary");
        j.set("exact_exponent", true);          // f_i is the real number base^(-2i/dims), rounded once
    }
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

    Json blocks = Json::array(), order = Json::array();
    const Json& layers = c.get("layers");
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& l = layers.at(i);
        const Json& mx = l.get("mixer");
        const std::string kind = l.get("type").as_string();
        Json mixer = Json::object();
        mixer.set("hidden_size", width);
        mixer.set("num_heads", mx.get("heads").as_int());
        mixer.set("head_dim", mx.get("dim").as_int());
        mixer.set("value_dim", mx.get("vdim").as_int());
        if (kind == "mlstm") {
            mixer.set("kind", "gated_memory");
            mixer.set("gate_cap", mx.get("gate_cap").as_double());
            mixer.set("eps", eps);
            mixer.set("gate", "sigmoid");
        } else if (kind == "latent_attention") {
            mixer.set("kind", "latent_attention");
            mixer.set("rot_dim", mx.get("rot_dim").as_int());
            mixer.set("kv_rank", mx.get("kv_rank").as_int());
            mixer.set("q_rank", mx.get("q_rank").as_int());
            mixer.set("scale", mx.get("scale").as_double());
            mixer.set("eps", eps);
            mixer.set("sink", true);
            mixer.set("gate", "sigmoid");
            mixer.set("position", rotary_part(mx.get("rot"), mx.get("rot_dim").as_int()));
        } else {
            mixer.set("kind", "attention");
            mixer.set("num_kv_heads", mx.get("kv_heads").as_int());
            mixer.set("scale", mx.get("scale").as_double());
            mixer.set("window", mx.get("mask").get("size").as_int());
            mixer.set("bias", true);
            mixer.set("score_maps", 2LL);
            mixer.set("combine_maps", true);
            mixer.set("lambda_init", mx.get("diff").as_double());
            mixer.set("combine_eps", eps);
            mixer.set("position", rotary_part(mx.get("rot"), mx.get("dim").as_int()));
            mixer.set("names", venizen::names_of({{"q", "q"}, {"k", "k"}, {"v", "v"}, {"o", "o"}, {"q_bias", "q.b"},
                                                  {"k_bias", "k.b"}, {"v_bias", "v.b"}, {"lq1", "lq1"}, {"lk1", "lk1"},
                                                  {"lq2", "lq2"}, {"lk2", "lk2"}}));
        }
        Json block = Json::object();
        block.set("kind", "parallel_block");
        Json names = Json::array();
        for (const char* n : {"", "mix.", "mlp."}) names.push(n);
        block.set("names", std::move(names));
        block.set("norm", layernorm_part(width, eps, "norm1"));
        block.set("mixer", std::move(mixer));
        if (!l.get("mlp").is_null()) {
            Json ffn = Json::object();
            ffn.set("kind", "dense_mlp");
            ffn.set("hidden_size", width);
            ffn.set("intermediate_size", l.get("mlp").get("ff").as_int());
            ffn.set("activation", "relu_squared");
            block.set("ffn", std::move(ffn));
        } else {
            block.set("ffn", nullptr);
        }
        Json layer = Json::object();
        layer.set("prefix", format("l%zu.", i));
        layer.set("part", std::move(block));
        blocks.push(std::move(layer));
        Json run = Json::object();
        run.set("layer", (long long)i);
        run.set("cache", (long long)i);
        run.set("writes_cache", true);
        order.push(std::move(run));
    }
    p.set("layers", std::move(blocks));
    p.set("order", std::move(order));

    Json fn = Json::object();
    fn.set("prefix", "");
    fn.set("part", layernorm_part(width, eps, "final.norm"));
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

}  // namespace varunex

inline void register_varunex() {
    Registry::get().add_architecture("Varunex", Architecture{varunex::normalize, varunex::plan});
}

}  // namespace kipp
