// Tikunex: its config.json, checked and completed, and how it turns into parts.
//
// config.json is nested: "vocab", "width", "norm": {"eps"}, "layers": a list of {"type", "mixer", "mlp"}, and optionally
// "loop": {"start", "stop", "times"} and "token_side": {"dim"}.  Every size and constant comes from there (two inner sizes
// of the decay projections come from the checkpoint's tensor shapes unless "decay_rank" names them).
//
// The model: token table, then the model's norm; layers in order, where the layers loop.start .. loop.stop-1 run
// loop.times times in a row with the same weights and a cache entry of their own each time, and right before each such
// pass x <- W_in [x; x0] (x0: the embedding's output); final norm; head.  A layer is a pre-norm block: a mixer
// ("gla": gated linear attention; "parallel": softmax attention without position encoding, behind a sliding window
// that keeps a sequence's first tokens in sight, side by side with token-shift decay mixing), routed experts (or no
// feed-forward), and a per-layer token input.  Norms keep their weight around zero (the multiplier is 1 + w).  The
// residual stream is 32-bit floats whatever the activations' dtype.
#include "friday/config.h"
#include "friday/parts.h"

namespace friday {

namespace {
const char* kName = "Tikunex";

const Json& member(const Json& d, const std::string& key, const std::string& where) {
    const Json* v = d.is_object() ? d.find(key) : nullptr;
    if (!v || v->is_null()) throw ConfigError("config.json: " + where + " needs '" + key + "'");
    return *v;
}

int64_t positive_int(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = member(d, key, where);
    if (!v.is_int() || v.as_int() <= 0) throw ConfigError("config.json: " + where + "'" + key + "' must be a positive integer");
    return v.as_int();
}

double number(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = member(d, key, where);
    if (!v.is_number()) throw ConfigError("config.json: " + where + "'" + key + "' must be a number");
    return v.as_double();
}

void check_gla(const Json& m, const std::string& where) {
    positive_int(m, "heads", where);
    positive_int(m, "dim", where);
    positive_int(m, "vdim", where);
    if (!(number(m, "tau", where) > 0)) throw ConfigError("config.json: " + where + "'tau' must be positive");
}

void check_parallel(const Json& m, const std::string& where) {
    const Json& left = member(m, "left", where);
    const std::string lw = where + "left: ";
    const int64_t heads = positive_int(left, "heads", lw), kv = positive_int(left, "kv_heads", lw);
    if (heads % kv) throw ConfigError(format("config.json: %s%lld heads cannot share %lld key/value heads", lw.c_str(), (long long)heads, (long long)kv));
    positive_int(left, "dim", lw);
    positive_int(left, "vdim", lw);
    number(left, "scale", lw);
    const Json& mask = member(left, "mask", lw);
    positive_int(mask, "size", lw + "mask: ");
    const Json& keep = member(mask, "keep_first", lw + "mask: ");
    if (!keep.is_int() || keep.as_int() < 0) throw ConfigError("config.json: " + lw + "mask: 'keep_first' must be an integer, not negative");
    const Json& right = member(m, "right", where);
    positive_int(right, "heads", where + "right: ");
    positive_int(right, "dim", where + "right: ");
    number(m, "left_scale", where);
    number(m, "right_scale", where);
}

void check_mlp(const Json& mlp, const std::string& where) {
    const std::string kind = member(mlp, "kind", where).as_string();
    if (kind != "moe") throw ConfigError("config.json: " + where + "feed-forward kind '" + kind + "' is not one this design has (moe)");
    positive_int(member(mlp, "expert", where), "ff", where + "expert: ");
    const Json& router = member(mlp, "router", where);
    const int64_t experts = positive_int(router, "experts", where + "router: "), top = positive_int(router, "top", where + "router: ");
    if (top > experts) throw ConfigError(format("config.json: %srouter: top %lld of %lld experts", where.c_str(), (long long)top, (long long)experts));
}

Json read_tikunex(const Json& d) {
    if (!d.is_object()) throw ConfigError("config.json: not an object");
    positive_int(d, "vocab", "");
    positive_int(d, "width", "");
    if (!(number(member(d, "norm", ""), "eps", "norm: ") > 0)) throw ConfigError("config.json: norm: 'eps' must be positive");
    const Json& layers = member(d, "layers", "");
    if (!layers.is_array() || layers.size() == 0) throw ConfigError("config.json: 'layers' must be a list of at least one layer");
    for (size_t i = 0; i < layers.size(); ++i) {
        const std::string where = format("layers[%zu]: ", i);
        const Json& type = member(layers[i], "type", where);
        const Json& mixer = member(layers[i], "mixer", where);
        if (type.as_string() == "gla") check_gla(mixer, where + "mixer: ");
        else if (type.as_string() == "parallel") check_parallel(mixer, where + "mixer: ");
        else throw ConfigError("config.json: " + where + "mixer type '" + type.as_string() + "' is not one this design has (gla, parallel)");
        const Json* mlp = layers[i].find("mlp");
        if (mlp && !mlp->is_null()) check_mlp(*mlp, where + "mlp: ");
    }
    const Json* loop = d.find("loop");
    if (loop && !loop->is_null()) {
        const Json& a = member(*loop, "start", "loop: ");
        const Json& b = member(*loop, "stop", "loop: ");
        const int64_t times = positive_int(*loop, "times", "loop: ");
        (void)times;
        if (!a.is_int() || !b.is_int() || a.as_int() < 0 || b.as_int() <= a.as_int() || b.as_int() > (int64_t)layers.size())
            throw ConfigError(format("config.json: loop: 0 <= start < stop <= %zu layers", layers.size()));
    }
    const Json* side = d.find("token_side");
    if (side && !side->is_null()) positive_int(*side, "dim", "token_side: ");
    Json v = d;                                   // complete as given; the names the registry looks for are added
    Json a = Json::array();
    a.push(Json(kName));
    v.set("architectures", a);
    v.set("architecture", Json(kName));
    return v;
}

PartSpec norm_spec(double eps, const std::string& tensor_name) {
    Json p = Json::object();
    p.set("eps", Json(eps));
    p.set("offset", Json(1.0));
    p.set("weight_name", Json(tensor_name));
    return PartSpec("rmsnorm", p, "");
}

void copy_rank(const Json& from, Json& to) {
    const Json* r = from.find("decay_rank");
    if (r && r->is_int() && r->as_int() > 0) to.set("decay_rank", *r);
}

PartSpec gla_spec(const Json& m, double eps) {
    Json p = Json::object();
    p.set("heads", m.at("heads"));
    p.set("dim", m.at("dim"));
    p.set("vdim", m.at("vdim"));
    p.set("tau", m.at("tau"));
    p.set("eps", Json(eps));
    copy_rank(m, p);
    return PartSpec("gated_linear_attention", p, "mix.");
}

PartSpec parallel_spec(const Json& m, double eps) {
    const Json& left = m.at("left");
    const Json& right = m.at("right");
    Json lp = Json::object();
    lp.set("n_heads", left.at("heads"));
    lp.set("n_kv_heads", left.at("kv_heads"));
    lp.set("head_dim", left.at("dim"));
    lp.set("v_head_dim", left.at("vdim"));
    lp.set("scale", left.at("scale"));
    lp.set("window", left.at("mask").at("size"));
    lp.set("keep_first", left.at("mask").at("keep_first"));
    lp.set("qkv_bias", Json(false));
    lp.set("out_bias", Json(false));
    Json names = Json::object();
    for (const char* n : {"q", "k", "v", "o"}) names.set(n, Json(n));
    lp.set("names", names);
    PartSpec ls("gqa_attention", lp, "left.");
    ls.parts["position"] = PartSpec("none");
    Json rp = Json::object();
    rp.set("heads", right.at("heads"));
    rp.set("dim", right.at("dim"));
    rp.set("eps", Json(eps));
    copy_rank(right, rp);
    PartSpec rs("shift_decay_mix", rp, "right.");
    Json pp = Json::object();
    Json members = Json::array(), scales = Json::array();
    members.push(Json("left"));
    members.push(Json("right"));
    scales.push(Json(m.at("left_scale").as_double()));
    scales.push(Json(m.at("right_scale").as_double()));
    pp.set("members", members);
    pp.set("scales", scales);
    PartSpec ps("parallel", pp, "mix.");
    ps.parts["left"] = ls;
    ps.parts["right"] = rs;
    return ps;
}

ModelSpec tikunex_spec(const Json& c) {
    ModelSpec spec;
    spec.architecture = kName;
    spec.vocab_size = c.at("vocab").as_int();
    spec.width = c.at("width").as_int();
    spec.max_positions = (int64_t)1 << 30;            // no position encoding: nothing bounds a sequence but the cache
    spec.embedding = "embed";
    spec.head = "head";
    spec.residual_f32 = true;
    const double eps = c.at("norm").at("eps").as_double();
    spec.embed_norm = norm_spec(eps, "embed.norm");
    spec.embed_norm.params.set("out", Json("float32"));
    spec.final_norm = norm_spec(eps, "final.norm");
    const Json& layers = c.at("layers");
    const int64_t n = (int64_t)layers.size();
    const Json* side = c.find("token_side");
    const int64_t side_dim = side && !side->is_null() ? side->at("dim").as_int() : 0;
    if (side_dim > 0) spec.shared["side.embed"] = {spec.vocab_size, n * side_dim};
    for (int64_t i = 0; i < n; ++i) {
        const Json& L = layers[(size_t)i];
        PartSpec block("prenorm", Json::object(), format("l%lld.", (long long)i));
        block.parts["norm1"] = norm_spec(eps, "norm1");
        block.parts["mixer"] = L.at("type").as_string() == "gla" ? gla_spec(L.at("mixer"), eps) : parallel_spec(L.at("mixer"), eps);
        const Json* mlp = L.find("mlp");
        if (mlp && !mlp->is_null()) {
            block.parts["norm2"] = norm_spec(eps, "norm2");
            Json p = Json::object();
            p.set("experts", mlp->at("router").at("experts"));
            p.set("top", mlp->at("router").at("top"));
            p.set("inner", mlp->at("expert").at("ff"));
            block.parts["feed_forward"] = PartSpec("routed_experts", p, "mlp.");
        } else {
            spec.ignorable.push_back(format("l%lld.norm2", (long long)i));       // a checkpoint may carry it all the same
        }
        if (side_dim > 0) {
            Json p = Json::object();
            p.set("dim", Json(side_dim));
            p.set("slice", Json(i));
            p.set("eps", Json(eps));
            p.set("table", Json("side.embed"));
            block.parts["token_input"] = PartSpec("gated_token_table", p, "side.");
        }
        spec.layers.push_back(block);
    }
    // the run order: every call has a cache entry of its own; the first layer of each pass of the loop takes the
    // injection
    const Json* loop = c.find("loop");
    int64_t a = n, b = n, times = 1;
    if (loop && !loop->is_null()) {
        a = loop->at("start").as_int();
        b = loop->at("stop").as_int();
        times = loop->at("times").as_int();
        spec.injections.push_back(Injection{"loop.in"});
    }
    auto call = [&](int64_t layer, bool inject) {
        LayerCall cl;
        cl.layer = (int)layer;
        cl.cache = (int)spec.program.size();
        cl.inject = inject ? 0 : -1;
        spec.program.push_back(cl);
    };
    for (int64_t i = 0; i < a; ++i) call(i, false);
    for (int64_t t = 0; t < times; ++t)
        for (int64_t i = a; i < b; ++i) call(i, i == a);
    for (int64_t i = b; i < n; ++i) call(i, false);
    return spec;
}

struct RegisterTikunex {
    RegisterTikunex() { register_architecture({kName, read_tikunex, tikunex_spec}); }
} register_tikunex;
}  // namespace

}  // namespace friday
