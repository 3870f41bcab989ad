// Reader for AWQ checkpoints in the safetensors container (a little-endian u64 header length, a JSON header that
// maps tensor names to dtype / shape / byte range, then the raw tensor bytes).  The reference has no weight loader:
// it only leaves the hook, LayerParam::set_weight(idx, dims, ptr, device) (kuiper/source/op/layer.cpp:256-276), whose
// branch for quantised layers is empty there.  Here the file is memory-mapped, the tensors are handed to that hook
// as borrowed host pointers, and the model copies (and, under tensor parallelism, shards) them into its arena.
//
// Tensor names follow the Hugging Face layout of AWQ-quantised Qwen3 checkpoints:
//   model.embed_tokens.weight, model.norm.weight, lm_head.weight (optional: tied to the embedding when absent)
//   model.layers.<i>.input_layernorm.weight, .post_attention_layernorm.weight
//   model.layers.<i>.self_attn.{q,k}_norm.weight
//   model.layers.<i>.self_attn.{q,k,v,o}_proj.{qweight,qzeros,scales}
//   model.layers.<i>.mlp.{gate,up,down}_proj.{qweight,qzeros,scales}
// qweight I32 [in, out/8], qzeros I32 [in/group, out/8], scales F16 [in/group, out]; norms and tables BF16.
#ifndef KUIPER_INCLUDE_MODEL_CHECKPOINT_H
#define KUIPER_INCLUDE_MODEL_CHECKPOINT_H

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "base/base.h"

namespace model {

struct CheckpointTensor {
    std::string dtype;           // "I32", "F16", "BF16", "F32", ...
    std::vector<int64_t> shape;
    const unsigned char* data = nullptr;  // inside the mapping; valid while the file object lives
    size_t bytes = 0;
    int64_t element_count() const;
};

class SafetensorsFile : public base::NoCopyable {
public:
    ~SafetensorsFile();
    // maps `path` read-only and parses its header; every tensor's byte range is checked against the file size
    static base::Status open(const std::string& path, std::unique_ptr<SafetensorsFile>* out);
    // nullptr when the file has no tensor of that name
    const CheckpointTensor* find(const std::string& name) const;
    const std::map<std::string, CheckpointTensor>& tensors() const { return tensors_; }
    const std::map<std::string, std::string>& metadata() const { return metadata_; }

private:
    SafetensorsFile() = default;
    void* map_ = nullptr;
    size_t map_bytes_ = 0;
    std::map<std::string, CheckpointTensor> tensors_;
    std::map<std::string, std::string> metadata_;
};

}  // namespace model

#endif  // KUIPER_INCLUDE_MODEL_CHECKPOINT_H
