// Flat C handle API over the C++ host mirror, so that scripting languages
// (the Python package, tests) can drive the same graph engine.  Handles are
// heap-allocated katsu::Tensor / katsu::Conv2D objects; a Tensor handle is a
// strong reference to its node, like a Rust `Tensor` clone.
//
// Every function returns 0 on success or the katsu::ErrorKind value of the
// TensorError it caught; kh_last_error_* describe it.
#include <cstring>
#include <new>

#include "katsu.hpp"

using katsu::Conv2D;
using katsu::Tensor;
using katsu::TensorError;

namespace {

thread_local int g_kind = 0;
thread_local size_t g_a = 0, g_b = 0;
thread_local std::string g_message;

int record(const TensorError &e) {
    g_kind = static_cast<int>(e.kind);
    g_a = e.a;
    g_b = e.b;
    g_message = e.to_string();
    return g_kind;
}

int record_std(const std::exception &e) {
    g_kind = static_cast<int>(katsu::ErrorKind::Allocation);
    g_a = g_b = 0;
    g_message = std::string("tensor allocation failed: ") + e.what();
    return g_kind;
}

template <typename F>
int guarded(F &&body) {
    try {
        body();
        return 0;
    } catch (const TensorError &e) {
        return record(e);
    } catch (const std::exception &e) {
        return record_std(e);
    }
}

std::vector<size_t> shape_vec(const size_t *shape, size_t rank) { return std::vector<size_t>(shape, shape + rank); }

Tensor &T(void *h) { return *static_cast<Tensor *>(h); }
Conv2D &C(void *h) { return *static_cast<Conv2D *>(h); }
void *box(Tensor t) { return new Tensor(std::move(t)); }

struct GradBorrow {
    katsu::GradRef ref;
};

}  // namespace

extern "C" {

const char *kh_last_error_message(void) { return g_message.c_str(); }
void kh_last_error_numbers(size_t *a, size_t *b) {
    *a = g_a;
    *b = g_b;
}

int kh_set_device(int ordinal) {
    return guarded([&] { katsu::set_device(ordinal); });
}
int kh_set_precision(int mode) {
    return guarded([&] { katsu::set_precision(mode); });
}
int kh_synchronize(void) {
    return guarded([&] { katsu::synchronize(); });
}
int kh_context(void **out) {
    return guarded([&] { *out = katsu::device_context(); });
}
void kh_set_loss_fusion(int on) { katsu::set_loss_fusion(on != 0); }
int kh_loss_fusion(void) { return katsu::loss_fusion() ? 1 : 0; }

// ---- Tensor ---------------------------------------------------------------
int kh_tensor_new(const float *data, size_t len, const size_t *shape, size_t rank, void **out) {
    return guarded([&] {
        // Shape errors take precedence over copying a large payload.
        const std::vector<size_t> dims = shape_vec(shape, rank);
        const size_t expected = katsu::element_count(dims);
        if (expected != len) {
            TensorError e;
            e.kind = katsu::ErrorKind::DataLength;
            e.a = expected;
            e.b = len;
            throw e;
        }
        *out = box(Tensor::from_vec(std::vector<float>(data, data + len), dims));
    });
}

int kh_tensor_zeros(const size_t *shape, size_t rank, void **out) {
    return guarded([&] { *out = box(Tensor::zeros(shape_vec(shape, rank))); });
}

int kh_tensor_clone(void *h, void **out) {
    return guarded([&] { *out = box(T(h)); });
}

void kh_tensor_free(void *h) { delete static_cast<Tensor *>(h); }

size_t kh_tensor_rank(void *h) { return T(h).rank(); }
size_t kh_tensor_numel(void *h) { return T(h).numel(); }
void kh_tensor_shape(void *h, size_t *out) {
    const auto &s = T(h).shape();
    if (!s.empty()) memcpy(out, s.data(), s.size() * sizeof(size_t));
}
const void *kh_tensor_id(void *h) { return T(h).id(); }

int kh_tensor_data(void *h, float *out, size_t cap) {
    return guarded([&] {
        const auto &d = T(h).data();
        const size_t n = d.size() < cap ? d.size() : cap;
        if (n) memcpy(out, d.data(), n * sizeof(float));
    });
}

void kh_tensor_op(void *h, int *kind, size_t *stride, size_t *padding) {
    const katsu::Op op = T(h).op();
    *kind = op.kind;
    *stride = op.stride;
    *padding = op.padding;
}

void kh_tensor_op_flags(void *h, int *bias, int *relu) {
    const katsu::Op op = T(h).op();
    *bias = op.bias ? 1 : 0;
    *relu = op.relu ? 1 : 0;
}

size_t kh_tensor_parent_count(void *h) { return T(h).parents().size(); }
int kh_tensor_parent(void *h, size_t index, void **out) {
    return guarded([&] { *out = box(T(h).parents().at(index)); });
}

// Copies the gradient to `out` (up to cap floats); *has = 0 when grad is None.
int kh_tensor_grad(void *h, float *out, size_t cap, int *has) {
    return guarded([&] {
        katsu::GradRef ref = T(h).grad();
        *has = ref.has_value() ? 1 : 0;
        if (*has) {
            const auto &g = ref.value();
            const size_t n = g.size() < cap ? g.size() : cap;
            if (n) memcpy(out, g.data(), n * sizeof(float));
        }
    });
}

// A held borrow, like keeping the Ref guard of Tensor::grad alive.
int kh_tensor_borrow_grad(void *h, void **out) {
    return guarded([&] { *out = new GradBorrow{T(h).grad()}; });
}
void kh_grad_borrow_release(void *borrow) { delete static_cast<GradBorrow *>(borrow); }

int kh_tensor_zero_grad(void *h) {
    return guarded([&] { T(h).zero_grad(); });
}

int kh_tensor_add(void *a, void *b, void **out) {
    return guarded([&] { *out = box(T(a).add(T(b))); });
}
int kh_tensor_mul(void *a, void *b, void **out) {
    return guarded([&] { *out = box(T(a).mul(T(b))); });
}
int kh_tensor_sum(void *a, void **out) {
    return guarded([&] { *out = box(T(a).sum()); });
}
int kh_tensor_matmul(void *a, void *b, void **out) {
    return guarded([&] { *out = box(T(a).matmul(T(b))); });
}
int kh_tensor_reshape(void *a, const size_t *shape, size_t rank, void **out) {
    return guarded([&] { *out = box(T(a).reshape(shape_vec(shape, rank))); });
}
int kh_tensor_backward(void *a) {
    return guarded([&] { T(a).backward(); });
}
int kh_tensor_backward_with(void *a, const float *seed, size_t len) {
    return guarded([&] { T(a).backward_with(std::vector<float>(seed, seed + len)); });
}
int kh_tensor_sgd_step(void *a, float lr) {
    return guarded([&] { T(a).sgd_step(lr); });
}
int kh_tensor_to_device(void *a) {
    return guarded([&] { T(a).to_device(); });
}
int kh_tensor_to_host(void *a) {
    return guarded([&] { T(a).to_host(); });
}
int kh_tensor_device_data(void *a, const void **out) {
    return guarded([&] { *out = T(a).device_data(); });
}
int kh_tensor_device_grad(void *a, const void **out) {
    return guarded([&] { *out = T(a).device_grad(); });
}

// ---- Conv2D ---------------------------------------------------------------
int kh_conv_new_seeded(size_t in_channels, size_t out_channels, size_t kh, size_t kw, size_t stride, size_t padding,
                       uint64_t seed, void **out) {
    return guarded([&] {
        *out = new Conv2D(Conv2D::new_seeded(in_channels, out_channels, {kh, kw}, stride, padding, seed));
    });
}
int kh_conv_from_weights(void *weights, size_t stride, size_t padding, void **out) {
    return guarded([&] { *out = new Conv2D(Conv2D::from_weights(T(weights), stride, padding)); });
}
// bias may be NULL (no bias).
int kh_conv_from_weights_bias(void *weights, void *bias, size_t stride, size_t padding, int relu, void **out) {
    return guarded([&] {
        *out = new Conv2D(Conv2D::from_weights_bias(T(weights), bias ? T(bias) : Tensor(), stride, padding, relu != 0));
    });
}
// *out = NULL when the layer has no bias.
int kh_conv_bias(void *h, void **out) {
    return guarded([&] { *out = C(h).bias().defined() ? box(C(h).bias()) : nullptr; });
}
int kh_conv_relu(void *h) { return C(h).relu() ? 1 : 0; }
void kh_conv_free(void *h) { delete static_cast<Conv2D *>(h); }
int kh_conv_weights(void *h, void **out) {
    return guarded([&] { *out = box(C(h).weights()); });
}
size_t kh_conv_stride(void *h) { return C(h).stride(); }
size_t kh_conv_padding(void *h) { return C(h).padding(); }
int kh_conv_forward(void *h, void *input, void **out) {
    return guarded([&] { *out = box(C(h).forward(T(input))); });
}
int kh_conv_backward(void *h, void *grad_output, void **out_dx, void **out_dw) {
    return guarded([&] {
        auto [dx, dw] = C(h).backward(T(grad_output));
        *out_dx = box(std::move(dx));
        *out_dw = box(std::move(dw));
    });
}
// *out = NULL when no forward is cached.
int kh_conv_activation_map(void *h, void **out) {
    return guarded([&] {
        auto map = C(h).get_activation_map();
        *out = map ? box(*map) : nullptr;
    });
}
void kh_conv_clear_cache(void *h) { C(h).clear_cache(); }

}  // extern "C"
