// ArgmaxSampler: greedy choice on the device.
#include "sampler/argmax_sampler.h"

#include "op/kernel/kernel_interface.h"

namespace sampler {
void ArgmaxSampler::sample(const tensor::Tensor& logits, const tensor::Tensor& next, void* stream) const {
    kernel::get_argmax_kernel(device_type_)(logits, next, stream);
}
}  // namespace sampler
