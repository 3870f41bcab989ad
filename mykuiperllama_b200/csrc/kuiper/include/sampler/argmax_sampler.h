// Greedy sampler.  The reference globs a kuiper/source/sampler directory that is absent
// (CMakeLists.txt:87); this is the argmax it would hold.  Runs on the device: only the
// chosen ids ever cross to the host.
#ifndef KUIPER_INCLUDE_SAMPLER_ARGMAX_SAMPLER_H
#define KUIPER_INCLUDE_SAMPLER_ARGMAX_SAMPLER_H

#include "tensor/tensor.h"

namespace sampler {
class ArgmaxSampler {
public:
    explicit ArgmaxSampler(base::DeviceType device_type) : device_type_(device_type) {}
    // logits [M, vocab] Fp32 -> next [M] Int32; ties resolve to the lowest index
    void sample(const tensor::Tensor& logits, const tensor::Tensor& next, void* stream) const;

private:
    base::DeviceType device_type_;
};
}  // namespace sampler

#endif  // KUIPER_INCLUDE_SAMPLER_ARGMAX_SAMPLER_H
