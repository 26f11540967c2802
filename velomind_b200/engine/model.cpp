// A decoder model built from a plan: embedding, layers run in the plan's order, final norm, head.
// Nothing here names an architecture; the plan says which parts and which order.
#include "ops.h"

namespace vmb {

// ------------------------------------------------------------------------------------------------ StepContext
void* StepContext::take_tokens(long long cols, DType dtype) { return ws->take(static_cast<size_t>(T_cap) * cols * dtype_size(dtype)); }

void* StepContext::take(long long elements, DType dtype) { return ws->take(static_cast<size_t>(elements) * dtype_size(dtype)); }

KVView StepContext::kv() const {
    const std::pair<int, int> where = cache->book.where(run);
    if (where.first < 0) throw CacheError(format("schedule position %d has no key/value cache", run));
    KVView v;
    v.k_pages = cache->k_pages(where.first, where.second);
    v.v_pages = cache->v_pages(where.first, where.second);
    v.block_table = tables[where.first];
    v.table_width = table_widths[where.first];
    v.n_pages = cache->book.n_pages;
    v.owns = (*schedule)[run].cache_of < 0;
    return v;
}

float* StepContext::state() const {
    const auto& s = cache->state[run];
    return s ? static_cast<float*>(s->ptr) : nullptr;
}

int StepContext::state_floats() const { return cache->book.state_floats[run]; }

// ------------------------------------------------------------------------------------------------ Layer
Layer::Layer(const BlockSpec& s) : spec(s) {
    parts.mixer = build_part_as<Mixer>("mixer", s.mixer);
    parts.feed_forward = build_part_as<FeedForward>("feed_forward", s.feed_forward);
    parts.mixer_norm = build_part_as<Norm>("norm", s.mixer_norm);
    parts.feed_forward_norm = build_part_as<Norm>("norm", s.feed_forward_norm);
    block = build_arrangement(s.arrangement, json::Value(), parts);
}

std::vector<std::pair<std::string, Part*>> Layer::named_parts() const {
    auto sub = [&](const char* role) {
        auto it = spec.names.find(role);
        return spec.prefix + (it != spec.names.end() ? it->second : std::string(role) + ".");
    };
    return {{sub("mixer"), parts.mixer.get()},
            {sub("feed_forward"), parts.feed_forward.get()},
            {sub("mixer_norm"), parts.mixer_norm.get()},
            {sub("feed_forward_norm"), parts.feed_forward_norm.get()}};
}

// ------------------------------------------------------------------------------------------------ DecoderModel
DecoderModel::DecoderModel(ModelPlan p) : plan(std::move(p)) {
    plan.validate();
    embedding = build_part_as<Embedding>("embedding", plan.embedding);
    for (const BlockSpec& b : plan.blocks) layers.emplace_back(b);
    final_norm = build_part_as<Norm>("norm", plan.final_norm);
    head = build_part_as<Head>("head", plan.head);
}

std::vector<std::pair<std::string, Part*>> DecoderModel::named_parts() const {
    std::vector<std::pair<std::string, Part*>> out;
    out.emplace_back(plan.embedding_prefix, embedding.get());
    for (const Layer& l : layers)
        for (auto& np : l.named_parts()) out.push_back(np);
    out.emplace_back(plan.final_norm_prefix, final_norm.get());
    out.emplace_back(plan.head_prefix, head.get());
    return out;
}

WeightTable DecoderModel::weight_table() const {
    WeightTable table;
    for (const auto& np : named_parts())
        for (const auto& kv : np.second->weight_specs()) table[np.first + kv.first] = kv.second;
    return table;
}

void DecoderModel::bind(const HostTensors& tensors, DType dt, int dev, cudaStream_t stream) {
    if (dt != DType::F32 && dt != DType::BF16) throw KernelError("a model computes in float32 or bfloat16");
    BindContext bc(dt, stream);
    for (const auto& np : named_parts()) {
        Weights w;
        for (const auto& kv : np.second->weight_specs()) w[kv.first] = tensors.at(np.first + kv.first);
        np.second->bind(w, bc);
    }
    dtype = dt;
    device = dev;
}

bool DecoderModel::graph_safe() const {
    for (const auto& np : named_parts())
        if (!np.second->graph_safe()) return false;
    for (const Layer& l : layers)
        if (!l.block->graph_safe()) return false;
    return true;
}

std::vector<CacheNeed> DecoderModel::cache_needs() const {
    std::vector<CacheNeed> out;
    for (const ScheduleEntry& e : plan.schedule) out.push_back(e.cache_of >= 0 ? CacheNeed{} : layers[e.layer].parts.mixer->cache_need());
    return out;
}

std::vector<int> DecoderModel::cache_shares() const {
    std::vector<int> out;
    for (const ScheduleEntry& e : plan.schedule) out.push_back(e.cache_of);
    return out;
}

// Run the step's tokens through every layer of the schedule; float32 logits [R, vocab] at ctx.logit_rows.
void DecoderModel::forward(StepContext& ctx) {
    const long long hid = plan.hidden_size;
    ctx.hidden = plan.hidden_size;
    float* h = static_cast<float*>(ctx.take_tokens(hid, DType::F32));
    embedding->forward(ctx, ctx.tokens, h);
    void* pending = nullptr;
    for (size_t run = 0; run < plan.schedule.size(); ++run) {
        ctx.run = static_cast<int>(run);
        pending = layers[plan.schedule[run].layer].block->forward(ctx, h, pending);
    }
    ctx.run = -1;
    // Final norm and head on the wanted rows (plus `pending`, a product not yet added to the residual stream).  A step that
    // wants no logits (a prompt cut into several steps) has a bucket of its own, so it asks for nothing here.
    if (ctx.R > 0) {
        void* rows = ctx.take(static_cast<long long>(ctx.R_cap) * hid, ctx.act_dtype);
        final_norm->forward(ctx, h, pending, rows, ctx.logit_rows, ctx.R);
        head->forward(ctx, rows, ctx.logits);
        ctx.give(rows);
    }
    ctx.give(pending);
    ctx.give(h);
}

WeightTable weight_table(const ModelPlan& plan) { return DecoderModel(plan).weight_table(); }

std::shared_ptr<DecoderModel> load_model(const std::string& folder, DType dtype, const std::string& device) {
    const json::Value data = read_config_json(folder);
    const std::string where = folder + "/config.json";
    const PlanFunction plan_of = resolve_architecture(data, where);
    auto model = std::make_shared<DecoderModel>(plan_of(data, where));
    model->config = data;
    const HostTensors tensors = load_weights(folder, model->weight_table());
    const int dev = require_cuda(device);          // one clear refusal before the first tensor moves: there is no CPU fallback
    cudaStream_t stream = nullptr;
    ops::cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "creating a stream");
    try {
        model->bind(tensors, dtype, dev, stream);
    } catch (...) {
        cudaStreamDestroy(stream);
        throw;
    }
    cudaStreamDestroy(stream);
    return model;
}

}  // namespace vmb
