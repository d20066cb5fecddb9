// Layer wrappers: one object per operator launch of a network, with the interface of portDNN's
// tools/layer.h:49-310 (Layer::run / get_output / get_output_size, and the same constructor
// argument order per layer type), so that code which builds networks out of these layers compiles
// against this implementation.  A layer owns nothing: every pointer is device memory of the caller.
#ifndef PORTDNN_B200_TOOLS_LAYER_H_
#define PORTDNN_B200_TOOLS_LAYER_H_
#include <cstddef>

#include "portdnn/batchnorm/launch.h"
#include "portdnn/binaryop/launch.h"
#include "portdnn/conv2d/launch.h"
#include "portdnn/matmul/launch.h"
#include "portdnn/pointwise/launch.h"
#include "portdnn/pointwise/params.h"
#include "portdnn/pooling/launch.h"
#include "portdnn/softmax/launch.h"

namespace sycldnn {

/** Common part of every layer: where its result lives and how large it is. */
template <typename DType, typename Backend>
struct Layer {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  Backend& backend_;

  explicit Layer(Backend& b) : backend_(b), result_{}, result_size_{0} {}
  Layer(Backend& b, DeviceMem result, size_t result_size) : backend_(b), result_{result}, result_size_{result_size} {}
  virtual ~Layer() = default;

  virtual DeviceMem get_output() { return result_; }
  virtual size_t get_output_size() const { return result_size_; }
  virtual SNNStatus run() = 0;

 protected:
  DeviceMem result_;
  size_t result_size_;
};

/** conv2d::launch<DType, Forward> with the selector's algorithm (tools/layer.h:62-96). */
template <typename DType, typename Backend>
struct ConvolutionLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  conv2d::Conv2DParams params_;
  DeviceMem input_, filter_, workspace_;
  size_t workspace_size_;
  conv2d::Selector& selector_;

  ConvolutionLayer(conv2d::Conv2DParams const& params, DeviceMem const input, DeviceMem const weights, DeviceMem output,
                   DeviceMem workspace, size_t workspace_size, Backend& b, conv2d::Selector& selector)
      : Layer<DType, Backend>(b, output, conv2d::get_sizes<conv2d::conv_type::Forward>(params).output_size),
        params_{params},
        input_{input},
        filter_{weights},
        workspace_{workspace},
        workspace_size_{workspace_size},
        selector_{selector} {}

  SNNStatus run() override {
    return conv2d::launch<DType, conv2d::conv_type::Forward>(input_, filter_, this->result_, params_, selector_,
                                                            this->backend_, workspace_, workspace_size_);
  }
};

/** binaryop::launch<DType, Add>: bias[C] added to every pixel (tools/layer.h:98-125). */
template <typename DType, typename Backend>
struct BiasAddLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  binaryop::BinaryParams params_;
  DeviceMem input_, biases_;

  BiasAddLayer(binaryop::BinaryParams const& params, DeviceMem const input, DeviceMem const bias, DeviceMem output,
               Backend& b)
      : Layer<DType, Backend>(b, output, binaryop::internal::count(params.lhs_dims)),
        params_{params},
        input_{input},
        biases_{bias} {}

  SNNStatus run() override {
    return binaryop::launch<DType, binaryop::Add>(input_, biases_, this->result_, params_, this->backend_);
  }
};

/** batchnorm forward in training mode: also writes the running statistics (tools/layer.h:127-166). */
template <typename DType, typename Backend>
struct BatchNormTrainingLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  batchnorm::BatchNormParams params_;
  DeviceMem input_, beta_, gamma_, input_mean_, input_variance_, running_mean_, running_variance_;

  BatchNormTrainingLayer(batchnorm::BatchNormParams const& params, DeviceMem const input, DeviceMem const beta,
                         DeviceMem const gamma, DeviceMem const input_mean, DeviceMem const input_variance,
                         DeviceMem running_mean, DeviceMem running_variance, DeviceMem output, Backend& b)
      : Layer<DType, Backend>(b, output, size_t(params.batch) * params.rows * params.cols * params.channels),
        params_{params},
        input_{input},
        beta_{beta},
        gamma_{gamma},
        input_mean_{input_mean},
        input_variance_{input_variance},
        running_mean_{running_mean},
        running_variance_{running_variance} {}

  SNNStatus run() override {
    return batchnorm::launch<DType, Backend, batchnorm::Forward>(input_, beta_, gamma_, input_mean_, input_variance_,
                                                                running_mean_, running_variance_, this->result_,
                                                                params_, this->backend_);
  }
};

/** batchnorm forward with frozen statistics (tools/layer.h:168-203). */
template <typename DType, typename Backend>
struct BatchNormFrozenLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  batchnorm::BatchNormParams params_;
  DeviceMem input_, beta_, gamma_, mean_, variance_;

  BatchNormFrozenLayer(batchnorm::BatchNormParams const& params, DeviceMem const input, DeviceMem const beta,
                       DeviceMem const gamma, DeviceMem const mean, DeviceMem const variance, DeviceMem output,
                       Backend& b)
      : Layer<DType, Backend>(b, output, size_t(params.batch) * params.rows * params.cols * params.channels),
        params_{params},
        input_{input},
        beta_{beta},
        gamma_{gamma},
        mean_{mean},
        variance_{variance} {}

  SNNStatus run() override {
    return batchnorm::launch<DType, Backend, batchnorm::Forward>(input_, beta_, gamma_, mean_, variance_,
                                                                this->result_, params_, this->backend_);
  }
};

/** pointwise::launch<DType, ActivationType, Forward> (tools/layer.h:205-228). */
template <typename DType, typename Backend, template <typename> class ActivationType>
struct ActivationLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  pointwise::PointwiseParams params_;
  DeviceMem input_;

  ActivationLayer(pointwise::PointwiseParams const& params, DeviceMem const input, DeviceMem output, Backend& b)
      : Layer<DType, Backend>(b, output, size_t(params.size)), params_{params}, input_{input} {}

  SNNStatus run() override {
    return pointwise::launch<DType, ActivationType, pointwise::Forward>(input_, this->result_, size_t(params_.size),
                                                                       this->backend_);
  }
};

/** pooling::launch<DType, PoolingType, Forward> (tools/layer.h:230-256). */
template <typename DType, typename Backend, template <typename> class PoolingType>
struct PoolingLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  pooling::PoolingParams params_;
  DeviceMem input_;

  PoolingLayer(pooling::PoolingParams const& params, DeviceMem const input, DeviceMem output, Backend& b)
      : Layer<DType, Backend>(b, output, pooling::get_sizes<pooling::Forward>(params).output_size),
        params_{params},
        input_{input} {}

  SNNStatus run() override {
    return pooling::launch<DType, PoolingType, pooling::Forward>(input_, this->result_, params_, this->backend_);
  }
};

/** Fully connected: output[m, n] = beta * output + input[m, k] * weights[k, n] on the backend's
 * matmul (tools/layer.h:258-282). */
template <typename DType, typename Backend>
struct FCLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  matmul::MatmulParams params_;
  DeviceMem input_, weights_;

  FCLayer(matmul::MatmulParams const& p, DeviceMem const input, DeviceMem const weights, DeviceMem output, Backend& b)
      : Layer<DType, Backend>(b, output, size_t(p.n)), params_(p), input_{input}, weights_{weights} {}

  SNNStatus run() override {
    using ConstPointer = typename Backend::template pointer_type<DType const>;
    Event done = this->backend_.template matmul<false, false>(ConstPointer{input_}, ConstPointer{weights_},
                                                              this->result_, DType(params_.beta), params_.m, params_.k,
                                                              params_.n);
    return SNNStatus{done, StatusCode::OK};
  }
};

/** softmax::launch<DType, Forward> (tools/layer.h:284-310). */
template <typename DType, typename Backend>
struct SoftmaxLayer : Layer<DType, Backend> {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  softmax::SoftmaxParams params_;
  DeviceMem input_, workspace_;

  SoftmaxLayer(softmax::SoftmaxParams const& params, DeviceMem const input, DeviceMem workspace, DeviceMem output,
               Backend& b)
      : Layer<DType, Backend>(b, output, size_t(softmax::get_sizes(params).output_size)),
        params_{params},
        input_{input},
        workspace_{workspace} {}

  SNNStatus run() override {
    return softmax::launch<DType, softmax::Forward, Backend>(input_, workspace_, this->result_, params_, this->backend_);
  }
};

}  // namespace sycldnn
#endif
