// Attention whose keys and values are made from one small latent per token.
//
//   latent_attention   queries through a latent of their own: c_q = rmsnorm(W_dq h), q = W_uq c_q,
//                      laid out head by head as [dim plain, rot_dim rotated].  W_dkv h has
//                      kv_rank + rot_dim rows: the first kv_rank, RMS-normed, are the latent c; the
//                      rest, rotated, is one key part shared by all heads.  Per head the plain
//                      key is W_uk c and the value W_uv c; score = (q_plain . k_plain + q_rot .
//                      k_rot) * scale.  Options: a sink per head in the softmax's denominator, a
//                      sigmoid gate per head from a projection of the mixer's input, a window.
//
// Only c and the rotated key part are cached: one key row of kv_rank + rot_dim elements per token,
// no value pages.  The products with W_uk and W_uv are moved to the query's side of the sums:
// q_lat = W_uk^T q_plain (per head) meets c directly, score = q_lat . c + q_rot . k_rot, the
// weighted sum runs over c itself, and W_uv expands it afterwards.  A step's cost then does not
// grow with heads x context, and prompts, portions and decoded tokens take the same path.
// Every size, eps, scale and tensor name is a parameter of the plan.
#pragma once
#include "recurrent_parts.hpp"

namespace kipp {

class LatentAttentionMixer : public Mixer {
public:
    LatentAttentionMixer(const Json& j, const BuildContext& ctx) {
        hidden_ = (int)j.get("hidden_size").as_int();
        heads_ = (int)j.get("num_heads").as_int();
        dim_ = (int)j.get("head_dim").as_int();
        rot_ = (int)j.get("rot_dim").as_int();
        v_dim_ = (int)j.get_int("value_dim", dim_);
        kv_rank_ = (int)j.get("kv_rank").as_int();
        q_rank_ = (int)j.get("q_rank").as_int();
        eps_ = (float)j.get("eps").as_double();
        scale_ = (float)j.get_double("scale", 1.0 / std::sqrt((double)(dim_ + rot_)));
        out_scale_ = (float)j.get_double("output_scale", 1.0);
        window_ = (int)j.get_int("window", 0);
        sink_on_ = j.get_bool("sink", false);
        gate_ = gate_code(j.get_string("gate", "none"));
        position_ = make_position(j.get("position"), ctx);
        names_ = tensor_names(j, {{"dq", "dq"}, {"dq_norm", "dq.norm"}, {"uq", "uq"}, {"dkv", "dkv"}, {"dkv_norm", "dkv.norm"},
                                  {"uk", "uk"}, {"uv", "uv"}, {"sink", "sink"}, {"g", "g"}, {"o", "o"}});
        if (hidden_ <= 0 || heads_ <= 0 || dim_ <= 0 || rot_ < 0 || v_dim_ <= 0 || kv_rank_ <= 0 || q_rank_ <= 0 || window_ < 0)
            fail(KIPP_E_CONFIG, "latent_attention: sizes must be positive");
        if (gate_ == 1) fail(KIPP_E_CONFIG, "latent_attention: the gate is none or sigmoid");
        if (position_->rotary_dim() != rot_ || rot_ % 2)
            fail(KIPP_E_CONFIG, "latent_attention: the position encoding must rotate all rot_dim dims (an even number)");
        qh_ = dim_ + rot_;
        row_ = kv_rank_ + rot_;
        g_off_ = q_rank_ + kv_rank_ + rot_;
        cols1_ = g_off_ + (gate_ ? heads_ : 0);
        ld1_ = pad8(cols1_);
        q_rank_ld_ = pad8(q_rank_);
        ldq_ = pad8(heads_ * qh_);
    }
    static int pad8(int n) { return (n + 7) / 8 * 8; }
    void tensor_specs(const std::string& p, std::vector<TensorSpec>& out) const override {
        auto add = [&](const char* role, std::vector<int64_t> shape, const char* init = "normal") {
            TensorSpec s;
            s.name = p + names_.at(role);
            s.shape = std::move(shape);
            s.init = init;
            out.push_back(s);
        };
        add("dq", {q_rank_, hidden_});
        add("dq_norm", {q_rank_}, "near_one");
        add("uq", {heads_ * qh_, q_rank_});
        add("dkv", {row_, hidden_});
        add("dkv_norm", {kv_rank_}, "near_one");
        add("uk", {heads_ * dim_, kv_rank_});
        add("uv", {heads_ * v_dim_, kv_rank_});
        if (sink_on_) add("sink", {heads_});
        if (gate_) add("g", {heads_, hidden_});
        add("o", {hidden_, heads_ * v_dim_});
        position_->tensor_specs(p, out);
    }
    std::optional<PagedKVSpec> cache_spec() const override {
        PagedKVSpec s{1, row_, window_, kv_rank_, 0};
        s.values_in_keys = true;
        return s;
    }
    void bind(Binder& b, const std::string& p) override {
        dtype_ = b.compute_dtype();
        const size_t es = dtype_size(dtype_);
        // one matrix for the two down projections and the gate
        w_in_ = b.allocate((size_t)cols1_ * hidden_ * es, p + "dq_dkv_g");
        char* base = static_cast<char*>(w_in_);
        b.load(p + names_.at("dq"), base, dtype_, hidden_, q_rank_, hidden_);
        b.load(p + names_.at("dkv"), base + (size_t)q_rank_ * hidden_ * es, dtype_, hidden_, row_, hidden_);
        if (gate_) b.load(p + names_.at("g"), base + (size_t)g_off_ * hidden_ * es, dtype_, hidden_, heads_, hidden_);
        // rows of W_uq padded to a multiple of 8 elements (zeros beyond the latent's size)
        w_uq_ = b.allocate((size_t)heads_ * qh_ * q_rank_ld_ * es, p + names_.at("uq"));
        cuda_check(cudaMemset(w_uq_, 0, (size_t)heads_ * qh_ * q_rank_ld_ * es), "clearing a padded weight");
        b.load(p + names_.at("uq"), w_uq_, dtype_, q_rank_ld_, (int64_t)heads_ * qh_, q_rank_);
        // W_uk of every head transposed to [kv_rank, dim]: it multiplies the plain part of the query
        void* uk = b.allocate((size_t)heads_ * dim_ * kv_rank_ * es, p + names_.at("uk"));
        b.load(p + names_.at("uk"), uk, dtype_, kv_rank_, (int64_t)heads_ * dim_, kv_rank_);
        w_uk_t_ = b.allocate((size_t)heads_ * dim_ * kv_rank_ * es, p + names_.at("uk") + " transposed");
        b.ops().transpose_heads(w_uk_t_, uk, dtype_, heads_, dim_, kv_rank_);
        w_uv_ = b.allocate((size_t)heads_ * v_dim_ * kv_rank_ * es, p + names_.at("uv"));
        b.load(p + names_.at("uv"), w_uv_, dtype_, kv_rank_, (int64_t)heads_ * v_dim_, kv_rank_);
        ldo_ = pad8(heads_ * v_dim_);
        w_o_ = b.allocate((size_t)hidden_ * ldo_ * es, p + names_.at("o"));
        cuda_check(cudaMemset(w_o_, 0, (size_t)hidden_ * ldo_ * es), "clearing a padded weight");
        b.load(p + names_.at("o"), w_o_, dtype_, ldo_, hidden_, (int64_t)heads_ * v_dim_);
        dq_norm_ = load_f32(b, p + names_.at("dq_norm"), q_rank_);
        dkv_norm_ = load_f32(b, p + names_.at("dkv_norm"), kv_rank_);
        if (sink_on_) sink_ = load_f32(b, p + names_.at("sink"), heads_);
        position_->bind(b, p);
    }
    size_t weight_bytes() const override {
        return ((size_t)cols1_ * hidden_ + (size_t)heads_ * qh_ * q_rank_ + (size_t)heads_ * (dim_ + v_dim_) * kv_rank_ +
                (size_t)hidden_ * heads_ * v_dim_) * dtype_size(dtype_) + (size_t)(q_rank_ + kv_rank_ + heads_) * 4;
    }
    bool folds_rms() const override { return Ops::gemm_scale_ok(dtype_, w_in_, hidden_, w_in_, hidden_); }
    void forward(StepContext& ctx, const LayerRun& run, int mixer_slot, const void* h, float* residual) override {
        const int T = ctx.tokens();
        const size_t es = ctx.element();
        Ops& ops = *ctx.ops;
        const StepMeta& m = *ctx.meta;
        NormFold fold_in, fold_out;
        const PagedCacheView cache = ctx.cache_view(run, mixer_slot);
        const float* cos_sin = step_rope_table(ctx, *position_, false);
        const int write = (run.writes_cache ? 1 : 0) | (ctx.kv_round_bf16 && ctx.dtype == F32 ? 2 : 0);
        // -- the down projections and the gate; the two norms; the latent and the rotated key part into the pages
        void* proj = ctx.workspace->buffer("latent_proj", (size_t)T * ld1_ * es);
        ops.gemm(proj, ctx.dtype, ld1_, h, hidden_, w_in_, hidden_, dtype_, T, cols1_, hidden_, EPI_STORE,
                 fold_input(ctx, fold_in));
        void* cq = ctx.workspace->buffer("latent_q", (size_t)T * q_rank_ld_ * es);
        if (q_rank_ld_ != q_rank_) cuda_check(cudaMemsetAsync(cq, 0, (size_t)T * q_rank_ld_ * es, ctx.stream), "clearing the padding");
        HeadSegment seg[3];
        seg[0].src_off = 0; seg[0].heads = 1; seg[0].dim = q_rank_; seg[0].src_stride = q_rank_; seg[0].norm_w = dq_norm_;
        seg[0].target = 0; seg[0].dst = cq; seg[0].ld_dst = q_rank_ld_; seg[0].dst_stride = q_rank_;
        seg[1].src_off = q_rank_; seg[1].heads = 1; seg[1].dim = kv_rank_; seg[1].src_stride = kv_rank_;
        seg[1].norm_w = dkv_norm_; seg[1].target = 1; seg[1].dst_off = 0;
        seg[2].src_off = q_rank_ + kv_rank_; seg[2].heads = 1; seg[2].dim = rot_; seg[2].src_stride = rot_;
        seg[2].rot = rot_; seg[2].cos_sin = cos_sin; seg[2].target = 1; seg[2].dst_off = kv_rank_;
        ops.head_segments(proj, ld1_, ctx.dtype, seg, rot_ > 0 ? 3 : 2, &cache, row_, 0, 1, m.positions, m.entry_of_token, T,
                          write, eps_);
        // -- the queries: up projection, the plain part through W_uk^T, the rotated part turned
        void* q = ctx.workspace->buffer("latent_q_up", (size_t)T * ldq_ * es);
        ops.gemm(q, ctx.dtype, ldq_, cq, q_rank_ld_, w_uq_, q_rank_ld_, dtype_, T, heads_ * qh_, q_rank_ld_, EPI_STORE);
        void* ql = ctx.workspace->buffer("q", (size_t)T * heads_ * row_ * es);
        ops.head_matmul(ql, (long long)heads_ * row_, row_, q, ldq_, qh_, w_uk_t_, (long long)kv_rank_ * dim_, ctx.dtype, T,
                        kv_rank_, dim_, heads_);
        if (rot_ > 0) {
            HeadSegment r;
            r.src_off = dim_; r.heads = heads_; r.dim = rot_; r.src_stride = qh_; r.rot = rot_; r.cos_sin = cos_sin;
            r.target = 0; r.dst = ql; r.ld_dst = (long long)heads_ * row_; r.dst_off = kv_rank_; r.dst_stride = row_;
            ops.head_segments(q, ldq_, ctx.dtype, &r, 1, nullptr, 0, 0, 0, m.positions, m.entry_of_token, T, 0, eps_);
        }
        // -- scores against [c, k_rot], the weighted sum of c, the gate
        AttentionExtras extras;
        extras.sink = sink_;
        extras.values_in_keys = 1;
        if (gate_) { extras.gate = proj; extras.ld_gate = ld1_; extras.gate_off = g_off_; }
        void* lat = ctx.workspace->buffer("latent_out", (size_t)T * heads_ * kv_rank_ * es);
        ops.attention_mix(lat, ql, cache, ctx.dtype, nullptr, m.positions, m.entry_of_token, T, heads_, 1, row_, kv_rank_,
                          scale_, window_, 0, out_scale_, nullptr, 0, m.q_start, m.context_len, &extras);
        // -- W_uv per head, then the output projection
        void* attn = ctx.workspace->buffer("attn_out", (size_t)T * ldo_ * es);
        if (ldo_ != heads_ * v_dim_) cuda_check(cudaMemsetAsync(attn, 0, (size_t)T * ldo_ * es, ctx.stream), "clearing the padding");
        ops.head_matmul(attn, ldo_, v_dim_, lat, (long long)heads_ * kv_rank_, kv_rank_, w_uv_, (long long)v_dim_ * kv_rank_,
                        ctx.dtype, T, v_dim_, kv_rank_, heads_);
        const NormFold* emit = fold_emit(ctx, fold_out, hidden_);
        ops.gemm(residual, F32, hidden_, attn, ldo_, w_o_, ldo_, dtype_, T, hidden_, ldo_, EPI_ADD, emit);
        fold_emitted(ctx, emit, hidden_);
    }

private:
    int hidden_ = 0, heads_ = 0, dim_ = 0, rot_ = 0, v_dim_ = 0, kv_rank_ = 0, q_rank_ = 0, window_ = 0;
    int qh_ = 0, row_ = 0, g_off_ = 0, cols1_ = 0, ld1_ = 0, q_rank_ld_ = 0, ldq_ = 0, ldo_ = 0, gate_ = 0, dtype_ = BF16;
    bool sink_on_ = false;
    float eps_ = 0.f, scale_ = 1.f, out_scale_ = 1.f;
    std::unique_ptr<PositionEncoding> position_;
    std::map<std::string, std::string> names_;
    void *w_in_ = nullptr, *w_uq_ = nullptr, *w_uk_t_ = nullptr, *w_uv_ = nullptr, *w_o_ = nullptr;
    float *dq_norm_ = nullptr, *dkv_norm_ = nullptr, *sink_ = nullptr;
};

inline void register_latent_parts(Registry& r) {
    r.add_part_kind("latent_attention", [](const Json& j, const BuildContext& ctx) -> std::unique_ptr<Part> {
        return std::make_unique<LatentAttentionMixer>(j, ctx);
    });
}

}  // namespace kipp
