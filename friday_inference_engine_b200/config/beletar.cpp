// Beletar: its config.json, checked and completed, and how it turns into parts.
//
// config.json is nested: "vocab", "width", "embedding": {"scale"}, "norm": {"eps"}, "layers": a list of {"type", "mixer",
// "mlp"}, and optionally "loop": {"start", "stop", "times"}.  Every size and constant comes from there (the inner sizes of
// two-step projections come from the checkpoint's tensor shapes).
//
// The model: token rows times embedding.scale, as a 32-bit residual stream; layers in order, where the layers
// loop.start .. loop.stop-1 run loop.times times in a row with the same weights and a cache entry of their own each time,
// and right before every such pass but the first the embedding's output is added to the stream; layer norm; the token
// table again as the head.  A layer is a pre-norm block with layer norms (weight and bias): a mixer ("delta": the gated
// delta rule with a decay per head; "channel_delta": with a decay per head and key channel and two-step gate and decay
// projections; "latent_attention": softmax attention over a cached latent with a rotated key part shared by the heads,
// a sink in the softmax and a gate per head) and a gated feed-forward (or none).
#include "friday/config.h"
#include "friday/parts.h"

namespace friday {

namespace {
const char* kName = "Beletar";

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

void check_delta(const Json& m, const std::string& where) {
    const int64_t heads = positive_int(m, "heads", where), kv = positive_int(m, "kv_heads", where);
    if (heads % kv) throw ConfigError(format("config.json: %s%lld heads cannot share %lld query/key heads", where.c_str(), (long long)heads, (long long)kv));
    positive_int(m, "dim", where);
    positive_int(m, "vdim", where);
    const int64_t taps = positive_int(m, "conv", where);
    if (taps > 8) throw ConfigError("config.json: " + where + "'conv' is at most 8 taps");
}

void check_latent(const Json& m, const std::string& where) {
    positive_int(m, "heads", where);
    positive_int(m, "dim", where);
    positive_int(m, "vdim", where);
    positive_int(m, "kv_rank", where);
    const int64_t rd = positive_int(m, "rot_dim", where);
    number(m, "scale", where);
    const Json& rot = member(m, "rot", where);
    const std::string rw = where + "rot: ";
    if (!(number(rot, "base", rw) > 1.0)) throw ConfigError("config.json: " + rw + "'base' must be greater than 1");
    const int64_t dims = positive_int(rot, "dims", rw);
    if (dims > rd || dims % 2) throw ConfigError("config.json: " + rw + "'dims' must be even and at most the mixer's 'rot_dim'");
    const Json* sc = rot.find("scaling");
    if (sc && !sc->is_null())
        for (const char* k : {"factor", "original", "fast", "slow"})
            if (!(number(*sc, k, rw + "scaling: ") > 0)) throw ConfigError("config.json: " + rw + "scaling: '" + k + "' must be positive");
}

void check_mlp(const Json& mlp, const std::string& where) {
    const std::string kind = member(mlp, "kind", where).as_string();
    if (kind != "dense") throw ConfigError("config.json: " + where + "feed-forward kind '" + kind + "' is not one this design has (dense)");
    positive_int(mlp, "ff", where);
}

Json read_beletar(const Json& d) {
    if (!d.is_object()) throw ConfigError("config.json: not an object");
    positive_int(d, "vocab", "");
    positive_int(d, "width", "");
    if (!(number(member(d, "norm", ""), "eps", "norm: ") > 0)) throw ConfigError("config.json: norm: 'eps' must be positive");
    const Json* emb = d.find("embedding");
    if (emb && !emb->is_null()) number(*emb, "scale", "embedding: ");
    const Json& layers = member(d, "layers", "");
    if (!layers.is_array() || layers.size() == 0) throw ConfigError("config.json: 'layers' must be a list of at least one layer");
    for (size_t i = 0; i < layers.size(); ++i) {
        const std::string where = format("layers[%zu]: ", i);
        const std::string type = member(layers[i], "type", where).as_string();
        const Json& mixer = member(layers[i], "mixer", where);
        if (type == "delta" || type == "channel_delta") check_delta(mixer, where + "mixer: ");
        else if (type == "latent_attention") check_latent(mixer, where + "mixer: ");
        else throw ConfigError("config.json: " + where + "mixer type '" + type + "' is not one this design has (delta, channel_delta, latent_attention)");
        const Json* mlp = layers[i].find("mlp");
        if (mlp && !mlp->is_null()) check_mlp(*mlp, where + "mlp: ");
    }
    const Json* loop = d.find("loop");
    if (loop && !loop->is_null()) {
        const Json& a = member(*loop, "start", "loop: ");
        const Json& b = member(*loop, "stop", "loop: ");
        positive_int(*loop, "times", "loop: ");
        if (!a.is_int() || !b.is_int() || a.as_int() < 0 || b.as_int() <= a.as_int() || b.as_int() > (int64_t)layers.size())
            throw ConfigError(format("config.json: loop: 0 <= start < stop <= %zu layers", layers.size()));
    }
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
    p.set("weight_name", Json(tensor_name));
    return PartSpec("layernorm", p, "");
}

PartSpec delta_spec(const Json& m, double eps, bool per_channel) {
    Json p = Json::object();
    p.set("heads", m.at("heads"));
    p.set("qk_heads", m.at("kv_heads"));
    p.set("dim", m.at("dim"));
    p.set("vdim", m.at("vdim"));
    p.set("conv", m.at("conv"));
    p.set("eps", Json(eps));
    p.set("decay", Json(per_channel ? "channel" : "head"));
    p.set("gate", Json(per_channel ? "low_rank" : "full"));
    // optional: the inner sizes of the two-step projections, for drawing random weights (a checkpoint's shapes give them)
    for (const char* k : {"decay_rank", "gate_rank"}) {
        const Json* r = m.find(k);
        if (r && r->is_int() && r->as_int() > 0) p.set(k, *r);
    }
    return PartSpec("gated_delta", p, "mix.");
}

PartSpec latent_spec(const Json& m, double eps) {
    Json p = Json::object();
    for (const char* k : {"heads", "dim", "vdim", "kv_rank", "rot_dim", "scale"}) p.set(k, m.at(k));
    p.set("eps", Json(eps));
    PartSpec s("latent_attention", p, "mix.");
    const Json& rot = m.at("rot");
    Json rp = Json::object();
    rp.set("base", rot.at("base"));
    rp.set("dims", rot.at("dims"));
    const Json* sc = rot.find("scaling");
    if (sc && !sc->is_null()) rp.set("scaling", *sc);
    s.parts["position"] = PartSpec("rotary_pairs", rp, "");
    return s;
}

ModelSpec beletar_spec(const Json& c) {
    ModelSpec spec;
    spec.architecture = kName;
    spec.vocab_size = c.at("vocab").as_int();
    spec.width = c.at("width").as_int();
    spec.max_positions = (int64_t)1 << 30;            // nothing bounds a sequence but the cache
    spec.embedding = "embed";                         // also the head
    spec.residual_f32 = true;
    const Json* emb = c.find("embedding");
    spec.embed_scale = emb && !emb->is_null() ? emb->at("scale").as_double() : 1.0;
    const double eps = c.at("norm").at("eps").as_double();
    spec.final_norm = norm_spec(eps, "final.norm");
    const Json& layers = c.at("layers");
    const int64_t n = (int64_t)layers.size();
    for (int64_t i = 0; i < n; ++i) {
        const Json& L = layers[(size_t)i];
        PartSpec block("prenorm", Json::object(), format("l%lld.", (long long)i));
        block.parts["norm1"] = norm_spec(eps, "norm1");
        const std::string type = L.at("type").as_string();
        block.parts["mixer"] = type == "latent_attention" ? latent_spec(L.at("mixer"), eps) : delta_spec(L.at("mixer"), eps, type == "channel_delta");
        const Json* mlp = L.find("mlp");
        if (mlp && !mlp->is_null()) {
            block.parts["norm2"] = norm_spec(eps, "norm2");
            Json p = Json::object();
            p.set("inner", mlp->at("ff"));
            Json names = Json::object();
            for (const char* r : {"gate", "up", "down"}) names.set(r, Json(r));
            p.set("names", names);
            block.parts["feed_forward"] = PartSpec("swiglu", p, "mlp.");
        } else {
            spec.ignorable.push_back(format("l%lld.norm2", (long long)i));       // a checkpoint may carry them all the same
            spec.ignorable.push_back(format("l%lld.norm2.b", (long long)i));
        }
        spec.layers.push_back(block);
    }
    // the run order: every call has a cache entry of its own; the first layer of each pass of the loop but the first
    // takes the embedding's output
    const Json* loop = c.find("loop");
    int64_t a = n, b = n, times = 1;
    if (loop && !loop->is_null()) {
        a = loop->at("start").as_int();
        b = loop->at("stop").as_int();
        times = loop->at("times").as_int();
    }
    auto call = [&](int64_t layer, bool add_input) {
        LayerCall cl;
        cl.layer = (int)layer;
        cl.cache = (int)spec.program.size();
        cl.add_input = add_input;
        spec.program.push_back(cl);
    };
    for (int64_t i = 0; i < a; ++i) call(i, false);
    for (int64_t t = 0; t < times; ++t)
        for (int64_t i = a; i < b; ++i) call(i, t > 0 && i == a);
    for (int64_t i = b; i < n; ++i) call(i, false);
    return spec;
}

struct RegisterBeletar {
    RegisterBeletar() { register_architecture({kName, read_beletar, beletar_spec}); }
} register_beletar;
}  // namespace

}  // namespace friday
