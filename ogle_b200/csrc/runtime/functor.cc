#include "functor.h"

namespace ogle {
namespace functor {

void SSDBBoxDecoder::operator()(Context* ctx, const Tensor* prediction_tensor, const Tensor* anchor_tensor,
                                Tensor* decoded_tensor, const std::vector<float>& variances) {
    OGLE_CHECK(!prediction_tensor->is_host());
    OGLE_CHECK(!anchor_tensor->is_host());
    OGLE_CHECK(!decoded_tensor->is_host());
    const IntList& p = prediction_tensor->shape();
    const IntList& a = anchor_tensor->shape();
    const IntList& d = decoded_tensor->shape();
    OGLE_CHECK_EQ(p.size(), 3u);
    OGLE_CHECK_EQ(d.size(), 3u);
    OGLE_CHECK_EQ(a.size(), 2u);
    OGLE_CHECK_EQ(d[2], 4);
    OGLE_CHECK_EQ(p[2], 4);
    OGLE_CHECK_EQ(a[0], p[1]);
    OGLE_CHECK_EQ(a[1], 4);
    OGLE_CHECK_EQ(variances.size(), 4u);
    OGLE_CUDA_OK(ogle_cuda_ssd_decode(prediction_tensor->device<float>(), anchor_tensor->device<float>(),
                                      decoded_tensor->device<float>(), p[0], p[1], variances.data(), ctx->stream()));
}

}  // namespace functor
}  // namespace ogle
