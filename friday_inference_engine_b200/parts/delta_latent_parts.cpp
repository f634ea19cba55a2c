// Two more mixers: the gated delta rule (a decay per head, or per head and key channel) and softmax attention over a
// cached latent.
//
//   mixer "gated_delta"        q, k (qk_heads x dim) and v (heads x vdim) pass a short causal convolution and silu; q and k
//                              are made unit vectors per head (q times dim^-1/2); head h reads q/k head h / (heads / qk_heads);
//                              beta = sigmoid(Wb h); decay g = exp(-exp(A_log) softplus(a + dt_bias)) with a = Wa h (one per
//                              head) or a = Wa2 (Wa1 h) (one per head and key channel: "decay": "channel");
//                              S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q;
//                              o / rms_head(o) * norm * gate, gate = silu(Wg h) or sigmoid(Wg2 (Wg1 h)) ("gate": "low_rank");
//                              then Wo.  State per sequence: the convolution's last taps-1 inputs, then the heads' matrices.
//   mixer "latent_attention"   q = Wq h (heads x [dim | rot]); Wdkv h = [latent (rank) | key part (rot)]; the latent is
//                              RMS-normed; query and key parts of size rot are rotated by the position part (its first `dims` numbers, if fewer); per head the
//                              key is [Wuk latent | key part], the value Wuv latent; causal softmax with a sink per head in
//                              the denominator; every head's result times sigmoid(Wg h)_head; then Wo.  The cache keeps the
//                              normed latent and the rotated key part, nothing per head.
//
// The states, decays, betas, unit norms, scores and weights are fp32 (csrc/delta.cu, csrc/attention_latent.cu).  Every
// part adds into the residual stream that it is given, in that stream's dtype.
#include <math.h>
#include <stdlib.h>

#include <string>

#include "friday/ops.h"
#include "friday/parts.h"

namespace friday {

namespace {

Tensor columns(const Tensor& t, int64_t c0, int64_t n) {
    Tensor v = t;
    v.data = (char*)t.data + (size_t)c0 * dtype_size(t.dtype);
    v.shape[1] = n;
    return v;
}

int positive(const PartSpec& s, const char* key, const char* part) {
    const int64_t v = s.params.get_int(key, 0);
    if (v <= 0) throw ConfigError(format("%s needs a positive '%s'", part, key));
    return (int)v;
}

}  // namespace

// ------------------------------------------------------------------ gated delta rule
class GatedDelta : public Mixer {
public:
    GatedDelta(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        heads_ = positive(s, "heads", "gated_delta");
        qk_heads_ = (int)s.params.get_int("qk_heads", heads_);
        dk_ = positive(s, "dim", "gated_delta");
        dv_ = (int)s.params.get_int("vdim", dk_);
        taps_ = (int)s.params.get_int("conv", 1);
        eps_ = (float)s.params.get_double("eps", 1e-5);
        const std::string decay = s.params.get_string("decay", "head"), gate = s.params.get_string("gate", "full");
        if (decay != "head" && decay != "channel") throw ConfigError("gated_delta: 'decay' is \"head\" or \"channel\"");
        if (gate != "full" && gate != "low_rank") throw ConfigError("gated_delta: 'gate' is \"full\" or \"low_rank\"");
        per_channel_ = decay == "channel";
        low_rank_gate_ = gate == "low_rank";
        if (qk_heads_ <= 0 || heads_ % qk_heads_) throw ConfigError(format("gated_delta: %d heads cannot share %d query/key heads", heads_, qk_heads_));
        if (dv_ <= 0 || taps_ < 1 || taps_ > 8) throw ConfigError("gated_delta: 'vdim' must be positive and 'conv' between 1 and 8");
        if (dk_ > 256) throw ConfigError("gated_delta: at most 256 key channels per head");
        const int64_t w = e.width, qk = (int64_t)qk_heads_ * dk_, hv = (int64_t)heads_ * dv_;
        // one product for everything in the activation dtype: q, k, v (and the full gate)
        declare_stacked("w_in", 2 * qk + hv + (low_rank_gate_ ? 0 : hv), w);
        declare("q", {qk, w}).stack("w_in", 0);
        declare("k", {qk, w}).stack("w_in", qk);
        declare("v", {hv, w}).stack("w_in", 2 * qk);
        if (!low_rank_gate_) declare("g", {hv, w}).stack("w_in", 2 * qk + hv);
        // a convolution of one tap is a multiplier per channel and keeps no history
        declare_stacked("taps", 2 * qk + hv, taps_);
        declare("q.conv", {qk, (int64_t)taps_}).stack("taps", 0);
        declare("k.conv", {qk, (int64_t)taps_}).stack("taps", qk);
        declare("v.conv", {hv, (int64_t)taps_}).stack("taps", 2 * qk);
        // what enters the recurrence: beta (and the per-head decay) in one product whose result stays 32-bit
        declare_stacked("w_rec", heads_ + (per_channel_ ? 0 : heads_), w);
        declare("b", {(int64_t)heads_, w}).stack("w_rec", 0);
        if (!per_channel_) declare("a", {(int64_t)heads_, w}).stack("w_rec", heads_);
        // the inner sizes of the two-step projections are the checkpoint's to give unless "decay_rank" / "gate_rank" name them
        const int64_t decay_rank = s.params.get_int("decay_rank", -1) > 0 ? s.params.get_int("decay_rank", -1) : -1;
        const int64_t gate_rank = s.params.get_int("gate_rank", -1) > 0 ? s.params.get_int("gate_rank", -1) : -1;
        if (per_channel_) {
            declare("a1", {decay_rank, w});
            declare("a2", {(int64_t)heads_ * dk_, decay_rank});
        }
        if (low_rank_gate_) {
            declare("g1", {gate_rank, w});
            declare("g2", {hv, gate_rank});
        }
        declare("A_log", {(int64_t)heads_});
        declare("dt_bias", {per_channel_ ? (int64_t)heads_ * dk_ : (int64_t)heads_});
        declare("norm", {(int64_t)dv_}, false, true);
        declare("o", {w, hv});
    }
    CacheRequest cache_request() const override {
        const int64_t channels = 2 * (int64_t)qk_heads_ * dk_ + (int64_t)heads_ * dv_;
        return CacheRequest::state({(int64_t)(taps_ - 1) * channels + (int64_t)heads_ * dk_ * dv_}, DType::F32);
    }
    void finalize(Ops& ops) override {
        Mixer::finalize(ops);
        if (per_channel_ && tensor("a1").rows() != tensor("a2").cols()) throw ConfigError(prefix + ": the decay's two projections do not fit each other");
        if (low_rank_gate_ && tensor("g1").rows() != tensor("g2").cols()) throw ConfigError(prefix + ": the gate's two projections do not fit each other");
    }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, Norm*) override {
        const int64_t qk = (int64_t)qk_heads_ * dk_, hv = (int64_t)heads_ * dv_;
        Tensor x = ops.materialize(h);
        Tensor in = ops.linear(Rows(x), tensor("w_in"));
        Tensor rec = ops.linear(Rows(x), tensor("w_rec"), nullptr, nullptr, (int)DType::F32);
        Tensor b_raw = columns(rec, 0, heads_), a_raw, gate;
        if (per_channel_) a_raw = ops.linear(Rows(ops.linear(Rows(x), tensor("a1"))), tensor("a2"), nullptr, nullptr, (int)DType::F32);
        else a_raw = columns(rec, heads_, heads_);
        if (low_rank_gate_) gate = ops.linear(Rows(ops.linear(Rows(x), tensor("g1"))), tensor("g2"));
        else gate = columns(in, 2 * qk + hv, hv);
        Ops::DeltaSpec sp;
        sp.heads = heads_;
        sp.qk_heads = qk_heads_;
        sp.dk = dk_;
        sp.dv = dv_;
        sp.taps = taps_;
        sp.per_channel = per_channel_;
        sp.q_scale = 1.0f / sqrtf((float)dk_);
        sp.unit_eps = 1e-6f;
        sp.q_off = 0;
        sp.k_off = qk;
        sp.v_off = 2 * qk;
        Tensor qkv = ops.conv_silu_unit(in, tensor("taps"), sp, view, ctx);
        Tensor o = ops.delta_scan(qkv, a_raw, b_raw, tensor("A_log"), tensor("dt_bias"), sp, view, ctx);
        Tensor y = ops.head_norm_gate(o, gate, tensor("norm"), false, heads_, dv_, eps_, out_scale, x.dtype, ctx, low_rank_gate_);
        return PartOut(ops.linear_residual(Rows(y), tensor("o"), nullptr, residual));
    }

private:
    int heads_, qk_heads_, dk_, dv_, taps_;
    float eps_;
    bool per_channel_, low_rank_gate_;
};

// ------------------------------------------------------------------ attention over a cached latent
class LatentAttention : public Mixer {
public:
    LatentAttention(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        heads_ = positive(s, "heads", "latent_attention");
        dim_ = positive(s, "dim", "latent_attention");
        rot_ = (int)s.params.get_int("rot_dim", 0);
        vdim_ = (int)s.params.get_int("vdim", dim_);
        rank_ = positive(s, "kv_rank", "latent_attention");
        eps_ = (float)s.params.get_double("eps", 1e-5);
        scale_ = (float)s.params.get_double("scale", 1.0 / sqrt((double)(dim_ + rot_)));
        has_sink_ = s.params.get_bool("sink", true);
        has_gate_ = s.params.get_bool("head_gate", true);
        if (rot_ < 0 || rot_ % 2 || vdim_ <= 0) throw ConfigError("latent_attention: 'rot_dim' must be even and not negative, 'vdim' positive");
        if (rank_ > 512 || rot_ > 128) throw ConfigError("latent_attention: a latent of at most 512 and a rotated part of at most 128");
        if ((int64_t)rank_ * 8 * 4 > 48 * 1024 || (int64_t)dim_ * 8 * 4 > 48 * 1024) throw ConfigError("latent_attention: head sizes beyond what the per-head products stage");
        position_ = adopt("", build<Position>("position", s.part("position"), e));
        const int64_t w = e.width, qd = (int64_t)heads_ * (dim_ + rot_), kvd = (int64_t)rank_ + rot_;
        declare_stacked("w_in", qd + kvd + (has_gate_ ? heads_ : 0), w);
        declare("q", {qd, w}).stack("w_in", 0);
        declare("dkv", {kvd, w}).stack("w_in", qd);
        if (has_gate_) declare("g", {(int64_t)heads_, w}).stack("w_in", qd + kvd);
        declare("dkv.norm", {(int64_t)rank_}, false, true);
        declare("uk", {(int64_t)heads_ * dim_, (int64_t)rank_});
        declare("uv", {(int64_t)heads_ * vdim_, (int64_t)rank_});
        if (has_sink_) declare("sink", {(int64_t)heads_});
        declare("o", {w, (int64_t)heads_ * vdim_});
    }
    // one row [latent | key part] per position: the latent lies in the key pool, the rotated key part in the value pool
    CacheRequest cache_request() const override { return CacheRequest::kv(1, rank_, 0, rot_ > 0 ? rot_ : rank_, 0); }
    void finalize(Ops& ops) override {
        Mixer::finalize(ops);
        if (rot_ > 0) {
            if (!position_->pairs(&freq_, &mult_, &rot_dims_) || rot_dims_ > rot_ || rot_dims_ % 2)
                throw ConfigError(prefix + ": latent_attention needs a position part that rotates neighbouring pairs of at most its rotated size");
        }
    }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, Norm*) override {
        if (rot_ == 0) throw ConfigError("latent_attention without a rotated part is not built");
        const int64_t qd = (int64_t)heads_ * (dim_ + rot_), kvd = (int64_t)rank_ + rot_;
        Tensor x = ops.materialize(h);
        Tensor in = ops.linear(Rows(x), tensor("w_in"));
        Ops::LatentSpec sp;
        sp.heads = heads_;
        sp.dim = dim_;
        sp.rot = rot_;
        sp.rank = rank_;
        sp.vdim = vdim_;
        sp.scale = scale_;
        sp.eps = eps_;
        sp.rot_mult = mult_;
        sp.rot_dims = rot_dims_;
        sp.freq = freq_;
        sp.q_off = 0;
        sp.kv_off = qd;
        sp.gate_off = has_gate_ ? qd + kvd : -1;
        // queries against the cached rows: [W_uk,h^T q_h | rotated part] per head, fp32
        Tensor qf = ops.alloc(DType::F32, x.rows(), (int64_t)heads_ * kvd);
        Tensor ckr = ops.latent_prepare(in, tensor("dkv.norm"), sp, qf, ctx);
        ops.kv_store(ckr, 0, rank_, view, ctx);
        // prompts in bfloat16: keys and values expanded per head, products on the tensor cores (FRIDAY_LATENT_TC=0: never)
        const char* tc = getenv("FRIDAY_LATENT_TC");
        if (x.dtype == DType::BF16 && view.dtype == DType::BF16 && !ctx.decode && ctx.max_q_len >= 32 && (int)ctx.q_lens.size() == ctx.n_seqs &&
            dim_ % 8 == 0 && rot_ % 8 == 0 && vdim_ % 8 == 0 && rank_ % 8 == 0 && !(tc && tc[0] == '0')) {
            ops.rotate_pairs(in, ctx, freq_, mult_, heads_, dim_ + rot_, dim_, rot_dims_);
            Tensor mixed = ops.latent_attention_prompt(in, tensor("uk"), tensor("uv"), has_sink_ ? &tensor("sink") : nullptr, sp, view, ctx);
            return PartOut(ops.linear_residual(Rows(mixed), tensor("o"), nullptr, residual, out_scale));
        }
        ops.head_linear(in, 0, dim_ + rot_, tensor("uk"), true, qf, kvd, nullptr, 0, heads_, dim_, rank_, ctx);
        Tensor lat = ops.latent_attention(qf, has_sink_ ? &tensor("sink") : nullptr, sp, view, ctx);
        // values: W_uv,h times the head's weighted latent, times the head's gate
        Tensor mixed = ops.alloc(x.dtype, x.rows(), (int64_t)heads_ * vdim_);
        ops.head_linear(lat, 0, rank_, tensor("uv"), false, mixed, vdim_, has_gate_ ? &in : nullptr, sp.gate_off, heads_, rank_, vdim_, ctx);
        return PartOut(ops.linear_residual(Rows(mixed), tensor("o"), nullptr, residual, out_scale));
    }

private:
    int heads_, dim_, rot_, vdim_, rank_, rot_dims_ = 0;
    float eps_, scale_, mult_ = 1.0f;
    bool has_sink_, has_gate_;
    Position* position_;
    const float* freq_ = nullptr;
};

namespace {
PartRegistrar d1("mixer", "gated_delta", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new GatedDelta(s, e); });
PartRegistrar d2("mixer", "latent_attention", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new LatentAttention(s, e); });
}  // namespace

}  // namespace friday
