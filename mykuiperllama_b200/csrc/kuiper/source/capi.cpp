// C ABI of the engine (include/kuiper_llama.h): thin forwarding to model::Qwen3Model.
#include "kuiper_llama.h"

#include <cstring>
#include <string>

#include "model/checkpoint.h"
#include "model/qwen3.h"

namespace {
thread_local std::string g_error;

int fail(const base::Status& st) {
    g_error = st.get_err_msg();
    return st.get_err_code();
}

int done(const base::Status& st) { return st ? 0 : fail(st); }

model::Qwen3Model* as_model(kuiper_model* m) { return reinterpret_cast<model::Qwen3Model*>(m); }
}  // namespace

extern "C" {

const char* kuiper_llama_last_error(void) { return g_error.c_str(); }

kuiper_model* kuiper_model_create(const kuiper_model_config* cfg) {
    if (!cfg) {
        g_error = "null config";
        return nullptr;
    }
    model::ModelConfig c;
    c.layer_num = cfg->n_layers;
    c.dim = cfg->hidden;
    c.head_num = cfg->n_q_heads;
    c.kv_head_num = cfg->n_kv_heads;
    c.head_size = cfg->head_dim;
    c.hidden_dim = cfg->inter;
    c.vocab_size = cfg->vocab;
    c.group_size = cfg->group;
    c.max_seq_len = cfg->max_seq;
    c.max_batch = cfg->max_batch;
    c.max_rows = cfg->max_rows;
    c.eps = cfg->eps;
    c.rope_theta = cfg->rope_theta;
    c.act_mode = cfg->act_mode;
    c.tp_rank = cfg->tp_rank;
    c.tp_size = cfg->tp_size;
    auto* m = new model::Qwen3Model(c);
    base::Status st = m->init(base::DeviceType::DeviceCUDA);
    if (!st) {
        fail(st);
        delete m;
        return nullptr;
    }
    return reinterpret_cast<kuiper_model*>(m);
}

void kuiper_model_destroy(kuiper_model* model) { delete as_model(model); }

int kuiper_model_load_layer(kuiper_model* model, int layer, const kuiper_layer_weights* w, int on_device) {
    if (!model || !w) return fail(base::error::invalid_argument("null pointer"));
    model::RawLayerWeights r;
    r.input_norm = w->input_norm; r.post_norm = w->post_norm; r.q_norm = w->q_norm; r.k_norm = w->k_norm;
    r.qkv_qw = w->qkv_qw; r.qkv_qz = w->qkv_qz; r.qkv_s = w->qkv_s;
    r.o_qw = w->o_qw; r.o_qz = w->o_qz; r.o_s = w->o_s;
    r.gu_qw = w->gu_qw; r.gu_qz = w->gu_qz; r.gu_s = w->gu_s;
    r.down_qw = w->down_qw; r.down_qz = w->down_qz; r.down_s = w->down_s;
    return done(as_model(model)->load_layer(layer, r, on_device != 0));
}

int kuiper_model_load_globals(kuiper_model* model, const void* embed, const void* final_norm, const void* lm_head,
                              int on_device) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->load_globals(embed, final_norm, lm_head, on_device != 0));
}

int kuiper_model_load_checkpoint(kuiper_model* model, const char* path) {
    if (!model || !path) return fail(base::error::invalid_argument("null pointer"));
    return done(as_model(model)->load_checkpoint(path));
}

int kuiper_checkpoint_inspect(const char* path, char* report, size_t report_bytes) {
    if (!path) return fail(base::error::invalid_argument("null path"));
    std::unique_ptr<model::SafetensorsFile> f;
    base::Status st = model::SafetensorsFile::open(path, &f);
    if (!st) return fail(st);
    std::string text;
    for (const auto& kv : f->tensors()) {
        text += kv.first + " " + kv.second.dtype + " [";
        for (size_t i = 0; i < kv.second.shape.size(); i++) text += (i ? "," : "") + std::to_string(kv.second.shape[i]);
        text += "] " + std::to_string(kv.second.bytes) + "\n";
    }
    for (const auto& kv : f->metadata()) text += "__metadata__ " + kv.first + "=" + kv.second + "\n";
    if (report && report_bytes > 0) {
        const size_t n = text.size() < report_bytes - 1 ? text.size() : report_bytes - 1;
        std::memcpy(report, text.data(), n);
        report[n] = 0;
    }
    return int(f->tensors().size()) > 0 ? 0 : fail(base::error::model_parse_error("the file holds no tensors"));
}

int kuiper_tp_unique_id(void* out128) {
    if (!out128) return fail(base::error::invalid_argument("null pointer"));
    return done(parallel::Communicator::make_unique_id(out128));
}

int kuiper_model_init_tp(kuiper_model* model, const void* unique_id128) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->init_tensor_parallel(unique_id128));
}

int kuiper_model_tp_one_shot(kuiper_model* model) {
    if (!model) return 0;
    const parallel::Communicator* c = as_model(model)->communicator();
    return c && c->one_shot_enabled() ? 1 : 0;
}

int kuiper_model_tp_status(kuiper_model* model) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    const parallel::Communicator* c = as_model(model)->communicator();
    return done(c ? c->one_shot_status() : base::error::success());
}

int kuiper_model_predict(kuiper_model* model, const int32_t* tokens, const int32_t* pos, const int32_t* slot, int M,
                         int32_t* next, float* logits) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    base::Status st = as_model(model)->predict(tokens, pos, slot, M, next);
    if (st && logits) st = as_model(model)->read_logits(logits, M);
    return done(st);
}

int kuiper_model_prefill(kuiper_model* model, const int32_t* tokens, int n, int slot, int32_t* next) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->prefill(tokens, n, slot, next));
}

int kuiper_model_decode_begin(kuiper_model* model, const int32_t* tokens, const int32_t* pos, const int32_t* slot,
                              int B) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->decode_begin(tokens, pos, slot, B));
}

int kuiper_model_decode_step(kuiper_model* model, int n_steps) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->decode_step(n_steps));
}

int kuiper_model_decode_read(kuiper_model* model, int32_t* tokens, int B) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->decode_read(tokens, B));
}

int kuiper_model_decode_predict(kuiper_model* model, const int32_t* tokens, int B, int32_t* next) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->decode_predict(tokens, B, next));
}

int kuiper_model_kernels_per_step(kuiper_model* model) { return model ? as_model(model)->kernels_per_step() : 0; }

void* kuiper_model_stream(kuiper_model* model) { return model ? as_model(model)->stream() : nullptr; }

int kuiper_model_synchronize(kuiper_model* model) {
    if (!model) return fail(base::error::invalid_argument("null model"));
    return done(as_model(model)->synchronize());
}

}  // extern "C"
