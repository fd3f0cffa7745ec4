// C++ host mirror of katsu-core's public surface with device storage.
//
// The reference is a Rust crate (crates/katsu-core); this header restates its
// API one-to-one so that code written against katsu_core::{Tensor, Conv2D, Op,
// TensorError} reads the same here, while every arithmetic loop is replaced by
// a call through the C ABI of include/katsu_cuda.h.  There is no CPU
// arithmetic in this layer: a missing device or library is a TensorError of
// kind Device, never a silent fallback.
//
//   Rust                                   here
//   Tensor(Rc<TensorNode>)                 katsu::Tensor (shared_ptr<TensorNode>)      tensor.rs:98-107
//   Op                                     katsu::Op (+ Reshape, an addition)          tensor.rs:85-93
//   TensorError                            katsu::TensorError (+ Device)               tensor.rs:9-82
//   Conv2D                                 katsu::Conv2D                               conv2d.rs:14-154
//   Result<T, TensorError>                 C++ exception of type TensorError
//   Ref<Option<Vec<f32>>> from grad()      katsu::GradRef (borrow counted like RefCell)
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <vector>

struct katsu_cuda_ctx;

namespace katsu {

enum class ErrorKind : int {
    ShapeOverflow = 1,
    InvalidConv,
    MissingForward,
    NonScalarBackward,
    GradientBorrowed,
    DataLength,
    ShapeMismatch,
    RankMismatch,
    MatmulMismatch,
    Allocation,
    Device,  // addition: a CUDA / library failure (no counterpart in the CPU-only reference)
};

// tensor.rs:9-82.  `a` and `b` carry the two numbers of DataLength
// {expected, actual}, RankMismatch {left, right} and MatmulMismatch
// {left_columns, right_rows}; `detail` the &'static str of InvalidConv.
struct TensorError {
    ErrorKind kind;
    size_t a = 0, b = 0;
    std::string detail;
    std::string to_string() const;  // the reference's Display text
};

// tensor.rs:85-93 plus Reshape (the reference has no view op).
struct Op {
    enum Kind : int { Leaf = 0, Add, Mul, Matmul, Conv2D, Sum, Reshape };
    Kind kind = Leaf;
    size_t stride = 0, padding = 0;  // Conv2D only
    // Conv2D only, additions (docs/roadmap.md:18-26 names bias and ReLU as the next layer features):
    // the node's third parent is a bias of one value per output channel; the output went through max(., 0).
    bool bias = false, relu = false;
    bool operator==(const Op &o) const {
        return kind == o.kind && stride == o.stride && padding == o.padding && bias == o.bias && relu == o.relu;
    }
};

// Selects the device ordinal used by every tensor created afterwards in this
// process (default 0).  Must be called before the first device operation.
void set_device(int ordinal);
// The process-wide context (created on first use).  Throws Device errors.
katsu_cuda_ctx *device_context();
// Precision mode of the contraction kernels (KATSU_MODE_* of katsu_cuda.h).
void set_precision(int mode);
// Blocks until all queued device work is done.
void synchronize();
// Loss-graph fusion (default on).  When on, y.mul(&y) does not compute its values until somebody asks
// for them, sum() of such a node reads y once, and backward carries the adjoints of that sub-graph
// in symbolic form (a broadcast scalar for y*y, "2 * scalar * y" for y) that a convolution consumes
// directly and that is written out only if the gradient is read.  Values and gradients are the
// ones the reference's node-by-node evaluation gives (tensor.rs:226-247, 392-417); off evaluates
// node by node.
void set_loss_fusion(bool on);
bool loss_fusion();

size_t element_count(const std::vector<size_t> &shape);  // tensor.rs:127-138

class Tensor;
struct TensorNode;

// Shared device allocation; freed when the last owner drops it.
struct DeviceBuffer {
    float *ptr = nullptr;
    size_t count = 0;
    explicit DeviceBuffer(size_t count);  // zero-filled (zeros_buffer, tensor.rs:120-125)
    ~DeviceBuffer();
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
};

// Guard returned by Tensor::grad(): while alive, backward and zero_grad on the
// node fail with GradientBorrowed (RefCell semantics of tensor.rs:200-215).
class GradRef {
   public:
    GradRef(std::shared_ptr<TensorNode> node);
    ~GradRef();
    GradRef(GradRef &&other) noexcept;
    GradRef(const GradRef &) = delete;
    bool has_value() const;
    const std::vector<float> &value() const;  // host copy of the gradient
    void release();

   private:
    std::shared_ptr<TensorNode> node_;
};

class Tensor {
   public:
    Tensor() = default;
    // Tensor::new (tensor.rs:148-158): takes the data, checks the length.
    static Tensor from_vec(std::vector<float> data, const std::vector<size_t> &shape);
    static Tensor zeros(const std::vector<size_t> &shape);  // tensor.rs:160-167

    const std::vector<size_t> &shape() const;
    // Host view of the values; the first call after a device op copies them back.
    const std::vector<float> &data() const;
    size_t rank() const;
    size_t numel() const;
    Op op() const;
    const std::vector<Tensor> &parents() const;

    GradRef grad() const;     // tensor.rs:200-206
    void zero_grad() const;   // tensor.rs:208-215

    Tensor add(const Tensor &rhs) const;     // tensor.rs:217-219
    Tensor mul(const Tensor &rhs) const;     // tensor.rs:222-224
    Tensor sum() const;                      // tensor.rs:243-247
    Tensor matmul(const Tensor &rhs) const;  // tensor.rs:250-280
    // Addition: same flat data under a new shape; the VJP passes g through.
    Tensor reshape(const std::vector<size_t> &shape) const;

    void backward() const;                                 // tensor.rs:309-314
    void backward_with(const std::vector<float> &seed) const;  // tensor.rs:320-362
    // Addition (docs/roadmap.md:21-22): data -= lr * grad in place on the device, the one operation
    // that changes a tensor's values after construction.  Without a gradient (no backward yet, or
    // zero_grad since) it fails with a Device error and changes nothing.
    void sgd_step(float lr) const;

    // Explicit transfers of the device storage variant.
    const Tensor &to_device() const;  // uploads now instead of at first use
    const Tensor &to_host() const;    // fills the host mirror now
    // Device accessors for callers that stay on the GPU (benchmarks).
    const float *device_data() const;
    const float *device_grad() const;  // nullptr while grad is None

    const TensorNode *id() const { return node_.get(); }  // Rc::as_ptr, tensor.rs:282-284
    bool defined() const { return node_ != nullptr; }
    const std::shared_ptr<TensorNode> &node() const { return node_; }

    static Tensor make_node(std::shared_ptr<DeviceBuffer> data, std::vector<size_t> shape, Op op,
                            std::vector<Tensor> parents);  // Tensor::node, tensor.rs:182-190
    // A node whose values are p * p of its (single, repeated) parent p and are computed on first use.
    static Tensor make_lazy_square(const Tensor &parent);

   private:
    explicit Tensor(std::shared_ptr<TensorNode> node) : node_(std::move(node)) {}
    Tensor elementwise(const Tensor &rhs, Op::Kind kind) const;
    std::vector<Tensor> topological_order() const;  // tensor.rs:288-306
    std::shared_ptr<TensorNode> node_;
    friend class Conv2D;
};

// conv2d.rs:14-154
class Conv2D {
   public:
    Conv2D(size_t in_channels, size_t out_channels, std::pair<size_t, size_t> kernel_size, size_t stride,
           size_t padding);  // Conv2D::new, seed 42
    static Conv2D new_seeded(size_t in_channels, size_t out_channels, std::pair<size_t, size_t> kernel_size,
                             size_t stride, size_t padding, uint64_t seed);
    static Conv2D from_weights(Tensor weights, size_t stride, size_t padding);
    // Addition: a layer with a bias of one value per output channel (an undefined Tensor for none)
    // and, optionally, a ReLU behind it; both run in the convolution kernel's epilogue.
    static Conv2D from_weights_bias(Tensor weights, Tensor bias, size_t stride, size_t padding, bool relu);
    const Tensor &bias() const { return bias_; }
    bool relu() const { return relu_; }

    const Tensor &weights() const { return weights_; }
    size_t in_channels() const { return weights_.shape()[1]; }
    size_t out_channels() const { return weights_.shape()[0]; }
    std::pair<size_t, size_t> kernel_size() const { return {weights_.shape()[2], weights_.shape()[3]}; }
    size_t stride() const { return stride_; }
    size_t padding() const { return padding_; }

    Tensor forward(const Tensor &input);                               // conv2d.rs:95-115
    std::pair<Tensor, Tensor> backward(const Tensor &grad_output) const;  // conv2d.rs:119-138
    std::optional<Tensor> get_activation_map() const;                  // conv2d.rs:143-148
    void clear_cache();                                                // conv2d.rs:151-153

   private:
    Conv2D(Tensor weights, size_t stride, size_t padding, int)
        : weights_(std::move(weights)), stride_(stride), padding_(padding) {}
    Tensor weights_;
    Tensor bias_;  // undefined: no bias
    bool relu_ = false;
    size_t stride_ = 1, padding_ = 0;
    std::optional<std::pair<Tensor, Tensor>> last_forward_;
};

// Geometry::new (conv2d.rs:183-224): validation + output size, integer only.
struct Geometry {
    size_t batch, cin, cout, h, w, kh, kw, oh, ow, stride, padding;
    Geometry(const Tensor &input, const Tensor &weights, size_t stride, size_t padding);
    std::vector<size_t> output_shape() const { return {batch, cout, oh, ow}; }
};

}  // namespace katsu
