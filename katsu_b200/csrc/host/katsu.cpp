// Implementation of the host mirror declared in katsu.hpp.  Graph bookkeeping
// follows crates/katsu-core/src/tensor.rs and conv2d.rs line by line (cited at
// each function); every numeric loop of the reference is a C-ABI call here.
#include "katsu.hpp"

#include <cmath>
#include <unordered_map>
#include <unordered_set>

#include "katsu_cuda.h"

namespace katsu {

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
std::string TensorError::to_string() const {
    switch (kind) {
        case ErrorKind::InvalidConv: return "invalid Conv2D: " + detail;
        case ErrorKind::MissingForward: return "Conv2D backward requires a successful forward";
        case ErrorKind::NonScalarBackward: return "backward requires one element; use sum() or backward_with(seed)";
        case ErrorKind::GradientBorrowed: return "release gradient borrows before backward or zero_grad";
        case ErrorKind::ShapeOverflow: return "shape exceeds addressable tensor storage";
        case ErrorKind::DataLength:
            return "expected " + std::to_string(a) + " elements, got " + std::to_string(b);
        case ErrorKind::ShapeMismatch: return "elementwise operations require identical shapes (no broadcasting)";
        case ErrorKind::RankMismatch:
            return "matmul requires rank 2, got " + std::to_string(a) + " and " + std::to_string(b);
        case ErrorKind::MatmulMismatch:
            return "matmul inner dimensions differ: " + std::to_string(a) + " and " + std::to_string(b);
        case ErrorKind::Allocation: return "tensor allocation failed: " + detail;
        case ErrorKind::Device: return "device error: " + detail;
    }
    return "unknown error";
}

namespace {

[[noreturn]] void fail(ErrorKind kind, std::string detail = "", size_t a = 0, size_t b = 0) {
    TensorError e;
    e.kind = kind;
    e.a = a;
    e.b = b;
    e.detail = std::move(detail);
    throw e;
}

int g_ordinal = 0;
katsu_cuda_ctx *g_ctx = nullptr;
bool g_loss_fusion = true;

void check(int32_t rc) {
    if (rc == KATSU_OK) return;
    const char *msg = katsu_cuda_last_error_string();
    fail(rc == KATSU_ERR_ALLOC ? ErrorKind::Allocation : ErrorKind::Device, msg ? msg : "");
}

}  // namespace

void set_device(int ordinal) {
    if (g_ctx != nullptr && ordinal != g_ordinal)
        fail(ErrorKind::Device, "set_device must be called before the first device operation");
    g_ordinal = ordinal;
}

katsu_cuda_ctx *device_context() {
    if (g_ctx == nullptr) check(katsu_cuda_init(g_ordinal, &g_ctx));
    return g_ctx;
}

void set_precision(int mode) { check(katsu_cuda_set_precision(device_context(), mode)); }

void synchronize() { check(katsu_cuda_sync(device_context())); }

void set_loss_fusion(bool on) { g_loss_fusion = on; }
bool loss_fusion() { return g_loss_fusion; }

// tensor.rs:127-138
size_t element_count(const std::vector<size_t> &shape) {
    for (size_t d : shape)
        if (d == 0) return 0;
    size_t count = 1;
    for (size_t d : shape)
        if (__builtin_mul_overflow(count, d, &count)) fail(ErrorKind::ShapeOverflow);
    if (count > static_cast<size_t>(INTPTR_MAX) / sizeof(float)) fail(ErrorKind::ShapeOverflow);
    return count;
}

// ---------------------------------------------------------------------------
// storage
// ---------------------------------------------------------------------------
DeviceBuffer::DeviceBuffer(size_t n) : count(n) {
    if (n != 0) check(katsu_cuda_alloc(device_context(), n, &ptr));
}

DeviceBuffer::~DeviceBuffer() {
    if (ptr != nullptr && g_ctx != nullptr) katsu_cuda_free(g_ctx, ptr);
}

// tensor.rs:101-107, with the data Vec replaced by {host mirror, device buffer}.
// Values never change after construction, so either copy may be materialised
// lazily from the other.
// An adjoint (or a published gradient) of `numel` values that is either a dense device buffer or
// one of the two symbolic forms the loss sub-graph sum(y * y) produces.  A symbolic form stands for
// exactly the values the reference's node-by-node VJPs would have stored (tensor.rs:392-417):
//   Bcast   every element is scalar[0]                       (Sum VJP into a fresh adjoint)
//   Scaled  element i is t + t with t = fl(scalar[0] * source[i])   (both Mul edges of y * y into y's fresh adjoint)
// `scalar` is a private one-element copy, `source` the node's own immutable values.
struct Adjoint {
    enum Kind { Dense, Bcast, Scaled };
    Kind kind = Dense;
    size_t numel = 0;
    std::shared_ptr<DeviceBuffer> dense;   // Dense: null until first needed (then zeros)
    std::shared_ptr<DeviceBuffer> scalar;  // Bcast, Scaled
    std::shared_ptr<DeviceBuffer> source;  // Scaled

    // Writes the values out (a no-op for an allocated dense adjoint) and returns the buffer.
    float *to_dense() {
        if (kind == Dense) {
            if (!dense) dense = std::make_shared<DeviceBuffer>(numel);
            return dense->ptr;
        }
        auto buffer = std::make_shared<DeviceBuffer>(numel);
        if (numel) {
            if (kind == Bcast)
                check(katsu_cuda_bcast_acc(device_context(), buffer->ptr, scalar->ptr, numel));  // 0 + s
            else
                check(katsu_cuda_square_vjp(device_context(), buffer->ptr, source->ptr, scalar->ptr, numel, 0));
        }
        dense = std::move(buffer);
        kind = Dense;
        scalar.reset();
        source.reset();
        return dense->ptr;
    }
};

struct TensorNode {
    std::vector<size_t> shape;
    size_t numel = 0;
    Op op;
    std::vector<Tensor> parents;
    mutable std::vector<float> host;
    mutable bool host_valid = false;
    mutable std::shared_ptr<DeviceBuffer> dev;  // null until uploaded / computed
    // channels-innermost copy of the values for the wide-channel convolution kernels, written when a Conv2D
    // first reads this tensor as its input and reused by that layer's backward (values never change);
    // staged_mode is the precision mode it was written in
    mutable std::shared_ptr<DeviceBuffer> staged;
    mutable int staged_mode = -1;
    // values are parents[0] * parents[0], not computed yet (set by Tensor::mul when fusion is on)
    mutable bool lazy_square = false;
    mutable std::shared_ptr<DeviceBuffer> grad_dev;  // null == None (unless grad_sym holds it)
    mutable std::shared_ptr<Adjoint> grad_sym;       // a gradient still in symbolic form
    mutable std::vector<float> grad_host;
    mutable bool grad_host_valid = false;
    mutable int borrows = 0;

    const float *device() const {
        if (!dev) {
            auto buffer = std::make_shared<DeviceBuffer>(numel);
            if (lazy_square) {
                const float *p = parents[0].device_data();
                if (numel) check(katsu_cuda_mul(device_context(), p, p, buffer->ptr, numel));
                lazy_square = false;
            } else if (numel) {
                check(katsu_cuda_h2d(device_context(), buffer->ptr, host.data(), numel));
                check(katsu_cuda_sync(device_context()));
            }
            dev = std::move(buffer);
        }
        return dev->ptr;
    }

    const std::vector<float> &host_data() const {
        if (!host_valid) {
            const float *src = device();
            host.assign(numel, 0.f);
            if (numel) check(katsu_cuda_d2h(device_context(), host.data(), src, numel));
            host_valid = true;
        }
        return host;
    }

    bool has_grad() const { return grad_dev != nullptr || grad_sym != nullptr; }

    // The gradient as a dense device buffer (null while it is None).
    const std::shared_ptr<DeviceBuffer> &dense_grad() const {
        if (grad_sym) {
            grad_sym->to_dense();
            grad_dev = grad_sym->dense;
            grad_sym.reset();
        }
        return grad_dev;
    }
};

// ---------------------------------------------------------------------------
// GradRef
// ---------------------------------------------------------------------------
GradRef::GradRef(std::shared_ptr<TensorNode> node) : node_(std::move(node)) {
    node_->borrows += 1;
    try {
        if (node_->has_grad() && !node_->grad_host_valid) {
            const float *src = node_->dense_grad()->ptr;
            node_->grad_host.assign(node_->numel, 0.f);
            if (node_->numel) check(katsu_cuda_d2h(device_context(), node_->grad_host.data(), src, node_->numel));
            node_->grad_host_valid = true;
        }
    } catch (...) {
        node_->borrows -= 1;
        throw;
    }
}
GradRef::~GradRef() { release(); }
GradRef::GradRef(GradRef &&other) noexcept : node_(std::move(other.node_)) { other.node_.reset(); }
bool GradRef::has_value() const { return node_ && node_->has_grad(); }
const std::vector<float> &GradRef::value() const { return node_->grad_host; }
void GradRef::release() {
    if (node_) {
        node_->borrows -= 1;
        node_.reset();
    }
}

// ---------------------------------------------------------------------------
// Tensor
// ---------------------------------------------------------------------------
Tensor Tensor::from_vec(std::vector<float> data, const std::vector<size_t> &shape) {
    const size_t expected = element_count(shape);
    if (data.size() != expected) fail(ErrorKind::DataLength, "", expected, data.size());
    auto node = std::make_shared<TensorNode>();
    node->shape = shape;
    node->numel = expected;
    node->op = Op{};
    node->host = std::move(data);
    node->host_valid = true;
    return Tensor(std::move(node));
}

Tensor Tensor::zeros(const std::vector<size_t> &shape) {
    const size_t count = element_count(shape);
    std::vector<float> data;
    try {
        data.assign(count, 0.f);
    } catch (const std::exception &e) {
        fail(ErrorKind::Allocation, e.what());
    }
    return from_vec(std::move(data), shape);
}

// The staged copy of a convolution's input for the given geometry, written on first use; null when the
// shape's kernels read x directly.
static const float *staged_input(const Tensor &x, size_t n, size_t c, size_t h, size_t w, size_t k, size_t r, size_t s,
                                 size_t stride, size_t padding) {
    katsu_cuda_ctx *ctx = device_context();
    size_t floats = 0;
    check(katsu_cuda_conv2d_staged_floats(ctx, n, c, h, w, k, r, s, stride, padding, &floats));
    if (floats == 0) return nullptr;
    int32_t mode = 0;
    check(katsu_cuda_get_precision(ctx, &mode));
    const TensorNode &node = *x.node();
    if (!node.staged || node.staged->count != floats || node.staged_mode != mode) {
        auto buffer = std::make_shared<DeviceBuffer>(floats);
        check(katsu_cuda_conv2d_stage(ctx, x.device_data(), buffer->ptr, n, c, h, w));
        node.staged = std::move(buffer);
        node.staged_mode = mode;
    }
    return node.staged->ptr;
}

Tensor Tensor::make_node(std::shared_ptr<DeviceBuffer> data, std::vector<size_t> shape, Op op,
                         std::vector<Tensor> parents) {
    auto node = std::make_shared<TensorNode>();
    node->numel = data->count;
    node->shape = std::move(shape);
    node->op = op;
    node->parents = std::move(parents);
    node->dev = std::move(data);
    return Tensor(std::move(node));
}

const std::vector<size_t> &Tensor::shape() const { return node_->shape; }
const std::vector<float> &Tensor::data() const { return node_->host_data(); }
size_t Tensor::rank() const { return node_->shape.size(); }
size_t Tensor::numel() const { return node_->numel; }
Op Tensor::op() const { return node_->op; }
const std::vector<Tensor> &Tensor::parents() const { return node_->parents; }

GradRef Tensor::grad() const { return GradRef(node_); }

void Tensor::zero_grad() const {
    if (node_->borrows != 0) fail(ErrorKind::GradientBorrowed);
    node_->grad_dev.reset();
    node_->grad_sym.reset();
    node_->grad_host.clear();
    node_->grad_host_valid = false;
}

const Tensor &Tensor::to_device() const {
    node_->device();
    return *this;
}

const Tensor &Tensor::to_host() const {
    node_->host_data();
    return *this;
}

const float *Tensor::device_data() const { return node_->device(); }
const float *Tensor::device_grad() const { return node_->has_grad() ? node_->dense_grad()->ptr : nullptr; }

Tensor Tensor::make_lazy_square(const Tensor &parent) {
    auto node = std::make_shared<TensorNode>();
    node->numel = parent.numel();
    node->shape = parent.shape();
    node->op.kind = Op::Mul;
    node->parents = {parent, parent};
    node->lazy_square = true;
    return Tensor(std::move(node));
}

void Tensor::sgd_step(float lr) const {
    if (node_->borrows != 0) fail(ErrorKind::GradientBorrowed);
    if (!node_->has_grad()) fail(ErrorKind::Device, "sgd_step needs a gradient: run backward first");
    const float *gradient = node_->dense_grad()->ptr;
    float *values = const_cast<float *>(node_->device());
    if (numel()) check(katsu_cuda_sgd_step(device_context(), values, gradient, lr, numel()));
    node_->host_valid = false;  // the host mirror is refilled from the device on the next data()
}

// tensor.rs:226-240
Tensor Tensor::elementwise(const Tensor &rhs, Op::Kind kind) const {
    if (shape() != rhs.shape()) fail(ErrorKind::ShapeMismatch);
    // y * y: the values wait until somebody reads them; sum() and backward never need them stored
    if (kind == Op::Mul && g_loss_fusion && id() == rhs.id()) return make_lazy_square(*this);
    auto out = std::make_shared<DeviceBuffer>(numel());
    const float *a = node_->device();
    const float *b = rhs.node_->device();
    if (kind == Op::Add)
        check(katsu_cuda_add(device_context(), a, b, out->ptr, numel()));
    else
        check(katsu_cuda_mul(device_context(), a, b, out->ptr, numel()));
    Op op;
    op.kind = kind;
    return make_node(std::move(out), shape(), op, {*this, rhs});
}

Tensor Tensor::add(const Tensor &rhs) const { return elementwise(rhs, Op::Add); }
Tensor Tensor::mul(const Tensor &rhs) const { return elementwise(rhs, Op::Mul); }

// tensor.rs:243-247 (tree order on the device instead of a left fold)
Tensor Tensor::sum() const {
    auto out = std::make_shared<DeviceBuffer>(1);
    if (node_->lazy_square && !node_->dev)  // sum(p * p) in one pass over p, bit-identical to mul then sum
        check(katsu_cuda_sumsq(device_context(), node_->parents[0].device_data(), out->ptr, numel()));
    else
        check(katsu_cuda_sum(device_context(), node_->device(), out->ptr, numel()));
    Op op;
    op.kind = Op::Sum;
    return make_node(std::move(out), {}, op, {*this});
}

// tensor.rs:250-280
Tensor Tensor::matmul(const Tensor &rhs) const {
    if (rank() != 2 || rhs.rank() != 2) fail(ErrorKind::RankMismatch, "", rank(), rhs.rank());
    const size_t m = shape()[0], k = shape()[1], n = rhs.shape()[1];
    if (k != rhs.shape()[0]) fail(ErrorKind::MatmulMismatch, "", k, rhs.shape()[0]);
    const size_t count = element_count({m, n});
    auto out = std::make_shared<DeviceBuffer>(count);
    if (count != 0 && k != 0)
        check(katsu_cuda_matmul_fwd(device_context(), node_->device(), rhs.node_->device(), out->ptr, m, k, n));
    Op op;
    op.kind = Op::Matmul;
    return make_node(std::move(out), {m, n}, op, {*this, rhs});
}

Tensor Tensor::reshape(const std::vector<size_t> &new_shape) const {
    const size_t count = element_count(new_shape);
    if (count != numel()) fail(ErrorKind::DataLength, "", numel(), count);
    node_->device();
    Op op;
    op.kind = Op::Reshape;
    // Shares the parent's buffer: values are immutable, so aliasing is safe.
    return make_node(node_->dev, new_shape, op, {*this});
}

// tensor.rs:288-306: iterative DFS, parents before children, dedup by identity.
std::vector<Tensor> Tensor::topological_order() const {
    std::vector<Tensor> order;
    std::unordered_set<const TensorNode *> visited;
    std::vector<std::pair<Tensor, bool>> stack;
    stack.emplace_back(*this, false);
    while (!stack.empty()) {
        auto [node, expanded] = stack.back();
        stack.pop_back();
        if (expanded) {
            order.push_back(node);
            continue;
        }
        if (!visited.insert(node.id()).second) continue;
        stack.emplace_back(node, true);
        const auto &parents = node.parents();
        for (auto it = parents.rbegin(); it != parents.rend(); ++it) stack.emplace_back(*it, false);
    }
    return order;
}

// tensor.rs:309-314
void Tensor::backward() const {
    if (numel() != 1) fail(ErrorKind::NonScalarBackward);
    backward_with({1.0f});
}

namespace {

// Pending adjoints of one backward pass, one per reachable node (tensor.rs:328-331).  The reference
// zero-fills every one up front; here a dense adjoint is allocated (zero-filled) when it is first
// needed, and the loss sub-graph's adjoints stay symbolic (see Adjoint).
using Pending = std::unordered_map<const TensorNode *, Adjoint>;
// Parents whose pending adjoint has received a contribution in this pass.  A pending adjoint
// starts as zeros, so the first contribution of a convolution or matmul VJP may overwrite it
// (0 + v == v) instead of reading it back: the read-modify-write epilogue of the strided dX
// launches was four times slower than the plain store.
using Touched = std::unordered_set<const TensorNode *>;

bool is_square(const Tensor &node) {
    return node.op().kind == Op::Mul && node.parents()[0].id() == node.parents()[1].id();
}

// A private one-element copy of a device scalar (the original is an adjoint that may later be
// published as a gradient and accumulated into).
std::shared_ptr<DeviceBuffer> copy_scalar(const float *src) {
    auto out = std::make_shared<DeviceBuffer>(1);
    check(katsu_cuda_d2d(device_context(), out->ptr, src, 1));
    return out;
}

// Op::backward, tensor.rs:365-449: adds this node's contribution to the
// pending adjoint of each parent.  `own` is the node's own (complete) adjoint.
void op_backward(const Tensor &node, Adjoint &own, Pending &pending, Touched &touched) {
    katsu_cuda_ctx *ctx = device_context();
    const Op op = node.op();
    const auto &parents = node.parents();
    switch (op.kind) {
        case Op::Leaf:
            return;
        case Op::Conv2D: {
            const Tensor &x = parents[0], &w = parents[1];
            const auto &xs = x.shape(), &ws = w.shape();
            const size_t plane = node.numel() ? node.numel() / (node.shape()[0] * node.shape()[1]) : 0;
            // Upstream gradient of the convolution proper: a symbolic "2 * s * y" adjoint is consumed
            // as it is (the kernels scale their outputs); bias and ReLU first take their own VJP.
            const float *g = nullptr, *gscale = nullptr;
            float gfactor = 1.f;
            std::shared_ptr<DeviceBuffer> masked;
            if (own.kind == Adjoint::Scaled && !op.relu && !op.bias && x.id() != w.id()) {
                g = own.source->ptr;
                gscale = own.scalar->ptr;
                gfactor = 2.f;
            } else {
                g = own.to_dense();  // the bias and ReLU VJPs read the upstream gradient itself
            }
            if (op.bias) {
                const Tensor &b = parents[2];
                float *pb = pending.at(b.id()).to_dense();
                float *dg = nullptr;
                if (op.relu && node.numel()) {
                    masked = std::make_shared<DeviceBuffer>(node.numel());
                    dg = masked->ptr;
                }
                check(katsu_cuda_bias_relu_bwd(ctx, node.device_data(), g, dg, pb, node.shape()[0], node.shape()[1], plane,
                                               op.relu ? 1 : 0, touched.count(b.id()) ? 1 : 0));
                touched.insert(b.id());
                if (dg != nullptr) g = dg;
            } else if (op.relu && node.numel()) {
                masked = std::make_shared<DeviceBuffer>(node.numel());
                check(katsu_cuda_bias_relu_bwd(ctx, node.device_data(), g, masked->ptr, nullptr, node.shape()[0],
                                               node.shape()[1], plane, 1, 0));
                g = masked->ptr;
            }
            float *px = pending.at(x.id()).to_dense(), *pw = pending.at(w.id()).to_dense();
            if (x.id() != w.id()) {
                // backward_buffers + `pending[parent] += grad` (tensor.rs:374-390)
                const int acc_x = touched.count(x.id()) ? 1 : 0, acc_w = touched.count(w.id()) ? 1 : 0;
                const float *xs_staged = staged_input(x, xs[0], xs[1], xs[2], xs[3], ws[0], ws[2], ws[3], op.stride, op.padding);
                if (acc_x == acc_w) {
                    check(katsu_cuda_conv2d_bwd_staged(ctx, x.device_data(), xs_staged, w.device_data(), g, gscale, gfactor,
                                                       px, pw, xs[0], xs[1], xs[2], xs[3], ws[0], ws[2], ws[3], op.stride,
                                                       op.padding, acc_x));
                } else {
                    check(katsu_cuda_conv2d_bwd_staged(ctx, x.device_data(), xs_staged, w.device_data(), g, gscale, gfactor,
                                                       px, nullptr, xs[0], xs[1], xs[2], xs[3], ws[0], ws[2], ws[3],
                                                       op.stride, op.padding, acc_x));
                    check(katsu_cuda_conv2d_bwd_staged(ctx, x.device_data(), xs_staged, w.device_data(), g, gscale, gfactor,
                                                       nullptr, pw, xs[0], xs[1], xs[2], xs[3], ws[0], ws[2], ws[3],
                                                       op.stride, op.padding, acc_w));
                }
                touched.insert(x.id());
                touched.insert(w.id());
            } else {
                // Same node on both edges: sequential adds into one adjoint (tests/conv2d.rs:109-116).
                DeviceBuffer dx(x.numel()), dw(w.numel());
                check(katsu_cuda_conv2d_bwd(ctx, x.device_data(), w.device_data(), g, dx.ptr, dw.ptr, xs[0], xs[1],
                                            xs[2], xs[3], ws[0], ws[2], ws[3], op.stride, op.padding, 0));
                check(katsu_cuda_axpy_acc(ctx, px, dx.ptr, x.numel()));
                check(katsu_cuda_axpy_acc(ctx, pw, dw.ptr, w.numel()));
                check(katsu_cuda_sync(ctx));
                touched.insert(x.id());
            }
            return;
        }
        case Op::Add:
        case Op::Mul: {
            if (op.kind == Op::Mul && own.kind == Adjoint::Bcast && is_square(node)) {
                // q = y * y under a broadcast adjoint s: both edges add fl(s * y) into y's adjoint
                const Tensor &y = parents[0];
                Adjoint &target = pending.at(y.id());
                if (!touched.count(y.id())) {
                    y.device_data();
                    target.kind = Adjoint::Scaled;
                    target.scalar = own.scalar;
                    target.source = y.node()->dev;
                    target.dense.reset();
                } else if (node.numel()) {
                    check(katsu_cuda_square_vjp(ctx, target.to_dense(), y.device_data(), own.scalar->ptr, node.numel(), 1));
                }
                touched.insert(y.id());
                return;
            }
            const float *g = own.to_dense();
            // Both edges are visited even when they are the same node (tensor.rs:392-409).
            for (int side = 0; side < 2; ++side) {
                const Tensor &parent = parents[side], &other = parents[1 - side];
                float *target = pending.at(parent.id()).to_dense();
                if (op.kind == Op::Add)
                    check(katsu_cuda_axpy_acc(ctx, target, g, node.numel()));
                else
                    check(katsu_cuda_mul_acc(ctx, target, g, other.device_data(), node.numel()));
                touched.insert(parent.id());
            }
            return;
        }
        case Op::Sum: {
            const Tensor &parent = parents[0];
            Adjoint &target = pending.at(parent.id());
            const float *g = own.to_dense();
            if (g_loss_fusion && is_square(parent) && !touched.count(parent.id())) {
                // the adjoint of y * y is the broadcast of g[0]: kept as that one number
                target.kind = Adjoint::Bcast;
                target.scalar = copy_scalar(g);
                target.dense.reset();
            } else {
                check(katsu_cuda_bcast_acc(ctx, target.to_dense(), g, parent.numel()));
            }
            touched.insert(parent.id());
            return;
        }
        case Op::Reshape:
            check(katsu_cuda_axpy_acc(ctx, pending.at(parents[0].id()).to_dense(), own.to_dense(), node.numel()));
            touched.insert(parents[0].id());
            return;
        case Op::Matmul: {
            const Tensor &a = parents[0], &b = parents[1];
            const size_t m = a.shape()[0], k = a.shape()[1], n = b.shape()[1];
            if (node.numel() == 0 || k == 0) return;  // tensor.rs:421-423
            const float *g = own.to_dense();
            float *pa = pending.at(a.id()).to_dense(), *pb = pending.at(b.id()).to_dense();
            if (a.id() != b.id()) {
                const int acc_a = touched.count(a.id()) ? 1 : 0, acc_b = touched.count(b.id()) ? 1 : 0;
                if (acc_a == acc_b) {
                    check(katsu_cuda_matmul_bwd(ctx, a.device_data(), b.device_data(), g, pa, pb, m, k, n, acc_a));
                } else {
                    check(katsu_cuda_matmul_bwd(ctx, a.device_data(), b.device_data(), g, pa, nullptr, m, k, n, acc_a));
                    check(katsu_cuda_matmul_bwd(ctx, a.device_data(), b.device_data(), g, nullptr, pb, m, k, n, acc_b));
                }
            } else {
                check(katsu_cuda_matmul_bwd(ctx, a.device_data(), b.device_data(), g, pa, nullptr, m, k, n, 1));
                check(katsu_cuda_matmul_bwd(ctx, a.device_data(), b.device_data(), g, nullptr, pb, m, k, n, 1));
            }
            touched.insert(a.id());
            touched.insert(b.id());
            return;
        }
    }
}

}  // namespace

// tensor.rs:320-362
void Tensor::backward_with(const std::vector<float> &seed) const {
    if (seed.size() != numel()) fail(ErrorKind::DataLength, "", numel(), seed.size());
    katsu_cuda_ctx *ctx = device_context();
    const std::vector<Tensor> order = topological_order();
    Pending pending;
    for (const Tensor &node : order) pending[node.id()].numel = node.numel();
    if (numel() != 0) {
        check(katsu_cuda_h2d(ctx, pending.at(id()).to_dense(), seed.data(), numel()));
        check(katsu_cuda_sync(ctx));  // `seed` may be a temporary
    }
    Touched touched;
    touched.insert(id());  // the seed
    for (auto it = order.rbegin(); it != order.rend(); ++it) op_backward(*it, pending.at(it->id()), pending, touched);
    // All borrows are validated before any gradient changes (tensor.rs:341-350).
    for (const Tensor &node : order)
        if (node.node()->borrows != 0) fail(ErrorKind::GradientBorrowed);
    for (const Tensor &node : order) {
        TensorNode &n = *node.node();
        Adjoint &adjoint = pending.at(node.id());
        if (n.has_grad()) {
            // tensor.rs:353-356: old += new, element by element
            const float *add = adjoint.to_dense();
            check(katsu_cuda_axpy_acc(ctx, n.dense_grad()->ptr, add, n.numel));
        } else if (adjoint.kind == Adjoint::Dense) {
            adjoint.to_dense();  // a node nothing contributed to still gets Some(zeros)
            n.grad_dev = std::move(adjoint.dense);  // tensor.rs:357-359: the adjoint buffer becomes the gradient
        } else {
            n.grad_sym = std::make_shared<Adjoint>(std::move(adjoint));  // written out when somebody reads it
        }
        n.grad_host_valid = false;
    }
}

// ---------------------------------------------------------------------------
// Conv2D
// ---------------------------------------------------------------------------
namespace {

// conv2d.rs:156-166
void validate_weights(const std::vector<size_t> &shape, size_t stride) {
    bool has_zero = false;
    for (size_t d : shape) has_zero |= (d == 0);
    if (shape.size() != 4 || has_zero) fail(ErrorKind::InvalidConv, "weights must have positive OIHW dimensions");
    if (stride == 0) fail(ErrorKind::InvalidConv, "stride must be positive");
}

void check_padding(size_t padding) {
    size_t pad2;
    if (__builtin_mul_overflow(padding, size_t(2), &pad2)) fail(ErrorKind::ShapeOverflow);
}

}  // namespace

// conv2d.rs:183-224
Geometry::Geometry(const Tensor &input, const Tensor &weights, size_t stride_, size_t padding_) {
    validate_weights(weights.shape(), stride_);
    if (input.rank() != 4) fail(ErrorKind::InvalidConv, "input must be rank 4 (NCHW)");
    const auto &x = input.shape();
    const auto &k = weights.shape();
    if (x[1] != k[1] || x[2] == 0 || x[3] == 0)
        fail(ErrorKind::InvalidConv, "input channels must match weights; H and W must be positive");
    element_count({x[1], x[2], x[3]});
    size_t pad2;
    if (__builtin_mul_overflow(padding_, size_t(2), &pad2)) fail(ErrorKind::ShapeOverflow);
    auto output_dim = [&](size_t size, size_t kernel) -> size_t {
        size_t padded;
        if (__builtin_add_overflow(size, pad2, &padded)) fail(ErrorKind::ShapeOverflow);
        if (padded < kernel) fail(ErrorKind::InvalidConv, "kernel exceeds padded input");
        size_t out = (padded - kernel) / stride_;
        if (__builtin_add_overflow(out, size_t(1), &out)) fail(ErrorKind::ShapeOverflow);
        return out;
    };
    oh = output_dim(x[2], k[2]);
    ow = output_dim(x[3], k[3]);
    element_count({k[0], oh, ow});
    element_count({x[0], k[0], oh, ow});
    batch = x[0]; cin = x[1]; cout = k[0]; h = x[2]; w = x[3]; kh = k[2]; kw = k[3];
    stride = stride_; padding = padding_;
}

Conv2D::Conv2D(size_t in_channels, size_t out_channels, std::pair<size_t, size_t> kernel_size, size_t stride,
               size_t padding)
    : Conv2D(new_seeded(in_channels, out_channels, kernel_size, stride, padding, 42)) {}

// conv2d.rs:35-61
Conv2D Conv2D::new_seeded(size_t in_channels, size_t out_channels, std::pair<size_t, size_t> kernel_size,
                          size_t stride, size_t padding, uint64_t seed) {
    const std::vector<size_t> shape = {out_channels, in_channels, kernel_size.first, kernel_size.second};
    validate_weights(shape, stride);
    check_padding(padding);
    const size_t count = element_count(shape);
    const size_t fan_in = element_count({shape[1], shape[2], shape[3]});
    std::vector<float> data(count, 0.f);
    const float bound = 1.0f / std::sqrt(static_cast<float>(fan_in));
    uint64_t state = seed;
    for (float &value : data) {
        state += 0x9e3779b97f4a7c15ULL;  // SplitMix64
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
        z ^= z >> 31;
        const float uniform = static_cast<float>(z >> 40) / 16777216.0f;
        value = (2.0f * uniform - 1.0f) * bound;
    }
    return from_weights(Tensor::from_vec(std::move(data), shape), stride, padding);
}

// conv2d.rs:65-74
Conv2D Conv2D::from_weights(Tensor weights, size_t stride, size_t padding) {
    validate_weights(weights.shape(), stride);
    check_padding(padding);
    return Conv2D(std::move(weights), stride, padding, 0);
}

Conv2D Conv2D::from_weights_bias(Tensor weights, Tensor bias, size_t stride, size_t padding, bool relu) {
    Conv2D layer = from_weights(std::move(weights), stride, padding);
    if (bias.defined() && (bias.rank() != 1 || bias.shape()[0] != layer.out_channels()))
        fail(ErrorKind::InvalidConv, "bias must have one value per output channel");
    layer.bias_ = std::move(bias);
    layer.relu_ = relu;
    return layer;
}

// conv2d.rs:95-115
Tensor Conv2D::forward(const Tensor &input) {
    const Geometry geometry(input, weights_, stride_, padding_);
    const std::vector<size_t> shape = geometry.output_shape();
    auto out = std::make_shared<DeviceBuffer>(element_count(shape));
    if (out->count != 0) {
        // the input is read through its staged copy, which the backward pass of this layer finds again
        const float *staged = staged_input(input, geometry.batch, geometry.cin, geometry.h, geometry.w, geometry.cout,
                                           geometry.kh, geometry.kw, stride_, padding_);
        check(katsu_cuda_conv2d_fwd_staged(device_context(), input.device_data(), staged, weights_.device_data(),
                                           bias_.defined() ? bias_.device_data() : nullptr, out->ptr, geometry.batch,
                                           geometry.cin, geometry.h, geometry.w, geometry.cout, geometry.kh,
                                           geometry.kw, stride_, padding_, relu_ ? 1 : 0));
    }
    Op op;
    op.kind = Op::Conv2D;
    op.stride = stride_;
    op.padding = padding_;
    op.bias = bias_.defined();
    op.relu = relu_;
    std::vector<Tensor> parents = {input, weights_};
    if (bias_.defined()) parents.push_back(bias_);
    Tensor output = Tensor::make_node(std::move(out), shape, op, std::move(parents));
    last_forward_ = std::make_pair(input, output);  // only reached on success
    return output;
}

// conv2d.rs:119-138: returns fresh leaves, never touches .grad
std::pair<Tensor, Tensor> Conv2D::backward(const Tensor &grad_output) const {
    if (!last_forward_) fail(ErrorKind::MissingForward);
    const Tensor &input = last_forward_->first;
    const Tensor &output = last_forward_->second;
    if (grad_output.shape() != output.shape())
        fail(ErrorKind::InvalidConv, "grad_output must match the output NCHW shape");
    const Geometry geometry(input, weights_, stride_, padding_);
    const size_t expected = element_count(geometry.output_shape());
    if (grad_output.numel() != expected) fail(ErrorKind::DataLength, "", expected, grad_output.numel());
    auto dx = std::make_shared<DeviceBuffer>(input.numel());
    auto dw = std::make_shared<DeviceBuffer>(weights_.numel());
    const float *g = grad_output.device_data();
    std::shared_ptr<DeviceBuffer> masked;
    if (relu_ && expected != 0) {  // addition: the upstream gradient passes where the activation did
        masked = std::make_shared<DeviceBuffer>(expected);
        check(katsu_cuda_bias_relu_bwd(device_context(), output.device_data(), g, masked->ptr, nullptr, geometry.batch,
                                       geometry.cout, geometry.oh * geometry.ow, 1, 0));
        g = masked->ptr;
    }
    const float *staged = staged_input(input, geometry.batch, geometry.cin, geometry.h, geometry.w, geometry.cout,
                                       geometry.kh, geometry.kw, stride_, padding_);
    check(katsu_cuda_conv2d_bwd_staged(device_context(), input.device_data(), staged, weights_.device_data(), g, nullptr,
                                       1.f, dx->ptr, dw->ptr, geometry.batch, geometry.cin, geometry.h, geometry.w,
                                       geometry.cout, geometry.kh, geometry.kw, stride_, padding_, 0));
    return {Tensor::make_node(std::move(dx), input.shape(), Op{}, {}),
            Tensor::make_node(std::move(dw), weights_.shape(), Op{}, {})};
}

std::optional<Tensor> Conv2D::get_activation_map() const {
    if (!last_forward_) return std::nullopt;
    return last_forward_->second;
}

void Conv2D::clear_cache() { last_forward_.reset(); }

}  // namespace katsu
