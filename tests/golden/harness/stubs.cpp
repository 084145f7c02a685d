// the three armadillo-based legacy CPU kernels are unused on the Qwen3 path
#include "tensor.h"
namespace my_vllm {
void scale_inplace_cpu(float, const Tensor&, void*) { std::abort(); }
void softmax_inplace_cpu(const Tensor&, void*) { std::abort(); }
void softmax_inplace_cpu(const float*, size_t) { std::abort(); }
void scale_sum_kernel_cpu(const Tensor&, const Tensor&, const Tensor&, int, int, int, void*) { std::abort(); }
}
