// Define-by-run autograd and the neural-network layers of the dense-contraction
// path, mirroring the reference's host-side objects:
//   Variable / Node / Parameter   src/learn/neural_network/autograd.rs:191-306, 647-698
//   Layer / Forward               src/learn/neural_network/layer.rs:597-696
//   Conv2, Dense, MaxPool2, Relu, Flatten   layer.rs:842-1267
//   CrossEntropyLoss              src/learn/neural_network/criterion.rs:30-77
//   SGD                           src/learn/neural_network/optimizer.rs:344-428
// Every operator runs on the device through the C ABI.
#pragma once

#include <deque>
#include <functional>

#include "tensor.hpp"

namespace autograph {

struct Node;

// An edge computes the gradient of `input` from the gradient of the node that
// owns the edge (VariableBuilder::edge, autograd.rs:94-136).  `into` is either
// null or a pre-allocated destination the op may write (beta = 0) and return.
struct Edge {
    std::shared_ptr<Node> input;
    std::function<Tensor(const Tensor &output_grad, Tensor *into)> op;
};

struct Node {
    Shape shape;
    ag_dtype dtype = AG_F32;
    bool has_grad = false;
    Tensor grad;           // set when has_grad; parameters pre-set storage in grad_storage
    Tensor grad_storage;   // optional: where the gradient must live (parameter bucket slice)
    int pending = 0;       // edges that will still deliver a gradient to this node
    std::vector<Edge> edges;
};

// Backward pass: breadth-first over nodes whose gradient is complete
// (Node::backward_grad, autograd.rs:239-261).  A second gradient arriving at a
// node is added to the first (autograd.rs:126-131).
inline void backward_from(const std::shared_ptr<Node> &root, const Tensor &grad) {
    if (root->has_grad) return;
    root->grad = grad;
    root->has_grad = true;
    std::deque<std::shared_ptr<Node>> queue;
    queue.push_back(root);
    while (!queue.empty()) {
        std::shared_ptr<Node> node = queue.front();
        queue.pop_front();
        std::vector<Edge> edges = std::move(node->edges);
        node->edges.clear();
        for (Edge &e : edges) {
            Node &in = *e.input;
            Tensor *into = (!in.has_grad && in.grad_storage.defined()) ? &in.grad_storage : nullptr;
            Tensor g = e.op(node->grad, into);
            if (g.shape() != in.shape || g.dtype() != in.dtype)
                throw Error(AG_ERR_SHAPE, "backward: gradient does not match its node");
            if (in.has_grad) {
                in.grad.scaled_add(1.f, g);
            } else {
                if (into && g.data() != into->data()) {
                    check(ag_copy(g.device(), into->data(), g.data(), g.nbytes()));
                    g = *into;
                }
                in.grad = g;
                in.has_grad = true;
            }
            if (--in.pending == 0) queue.push_back(e.input);
        }
    }
}

struct Variable {
    Tensor value;
    std::shared_ptr<Node> node;  // null: no gradient flows through this variable
};

// Builder of a variable with edges to its inputs (Variable::builder()).
class VariableBuilder {
   public:
    void edge(const std::shared_ptr<Node> &input,
              std::function<Tensor(const Tensor &, Tensor *)> op) {
        ++input->pending;
        edges_.push_back(Edge{input, std::move(op)});
    }
    Variable build(Tensor value) {
        Variable v;
        if (!edges_.empty()) {
            v.node = std::make_shared<Node>();
            v.node->shape = value.shape();
            v.node->dtype = value.dtype();
            v.node->edges = std::move(edges_);
        }
        v.value = std::move(value);
        return v;
    }

   private:
    std::vector<Edge> edges_;
};

// A trainable tensor: value, gradient slot and optimizer state
// (ParameterBase, autograd.rs:647-656).  Values, gradients and velocities of a
// model live in three flat buckets; a parameter holds views into them.
struct Parameter {
    Tensor value;
    Tensor grad;      // view into the gradient bucket
    Tensor velocity;  // view into the velocity bucket (SGD momentum state)
    std::shared_ptr<Node> node;  // set by init_grad() for the current step
    // ≙ Parameter::init_grad (autograd.rs:732-734)
    void init_grad() {
        node = std::make_shared<Node>();
        node->shape = value.shape();
        node->dtype = value.dtype();
        node->grad_storage = grad;
    }
    // ≙ Parameter::to_variable (autograd.rs:835-847)
    Variable to_variable() const { return Variable{value, node}; }
    bool has_grad() const { return node && node->has_grad; }
};

struct ConvOptions {
    int padding[2] = {0, 0}, stride[2] = {1, 1}, dilation[2] = {1, 1};
    bool is_default() const {
        return padding[0] == 0 && padding[1] == 0 && stride[0] == 1 && stride[1] == 1 &&
               dilation[0] == 1 && dilation[1] == 1;
    }
};

class Layer {
   public:
    virtual ~Layer() = default;
    // ≙ Forward::forward
    virtual Variable forward(Pool &pool, const Variable &input) = 0;
    // ≙ Layer::try_for_each_parameter
    virtual void parameters(std::vector<Parameter *> &) {}
    virtual const char *name() const = 0;
};

inline ag_conv2_options to_c_options(const Shape &filter, const ConvOptions &o) {
    ag_conv2_options c;
    c.filter[0] = (int32_t)filter[0];
    c.filter[1] = (int32_t)filter[1];
    for (int i = 0; i < 2; ++i) {
        c.padding[i] = o.padding[i];
        c.stride[i] = o.stride[i];
        c.dilation[i] = o.dilation[i];
    }
    return c;
}

// Conv2 (layer.rs:842-948, 1035-1047).  The device path of the reference is
// im2col -> dot -> permute -> bias; here one implicit-GEMM kernel does all of
// it, and the two backward edges are the matching implicit GEMMs.
class Conv2 : public Layer {
   public:
    Parameter weight;  // [outputs, inputs, fh, fw]
    bool has_bias = false;
    Parameter bias;    // [outputs]
    ConvOptions options;

    const char *name() const override { return "Conv2"; }
    void parameters(std::vector<Parameter *> &out) override {
        out.push_back(&weight);
        if (has_bias) out.push_back(&bias);
    }
    Variable forward(Pool &pool, const Variable &input) override {
        return forward_fused(pool, input, false, nullptr);
    }
    bool records_gradient(const Variable &input) const {
        return input.node || weight.node || (has_bias && bias.node);
    }
    // Forward with the following Relu (and 2-D max pool, window = stride) folded in.
    // Folding is only legal when no gradient is recorded: the backward edges of
    // Relu and MaxPool2 need the intermediate tensors.
    Variable forward_fused(Pool &pool, const Variable &input, bool relu, const int *pool_window) {
        const Tensor &x = input.value;
        if (x.ndim() != 4 || x.dim(1) != weight.value.dim(1))
            throw Error(AG_ERR_SHAPE, "Conv2: input channels do not match the weight");
        if (!x.is_standard_layout()) throw Error(AG_ERR_SHAPE, "Conv2 needs standard layout");
        const int64_t bs = x.dim(0), ic = x.dim(1), ih = x.dim(2), iw = x.dim(3);
        const int64_t oc = weight.value.dim(0);
        const Shape filter = {weight.value.dim(2), weight.value.dim(3)};
        const ag_conv2_options copt = to_c_options(filter, options);
        int64_t oh = 0, ow = 0;
        check(ag_conv2_output_shape(ih, iw, &copt, &oh, &ow));
        Variable w = weight.to_variable();
        Variable b = has_bias ? bias.to_variable() : Variable{};
        const bool needs_grad = input.node || w.node || b.node;
        if ((relu || pool_window) && needs_grad)
            throw Error(AG_ERR_INVALID, "Conv2: fused forward while a gradient is recorded");
        if (pool_window) {
            const int64_t ph = (oh - pool_window[0]) / pool_window[0] + 1;
            const int64_t pw = (ow - pool_window[1]) / pool_window[1] + 1;
            if (oh < pool_window[0] || ow < pool_window[1])
                throw Error(AG_ERR_SHAPE, "MaxPool2: window larger than input");
            Tensor y = Tensor::uninit(pool, {bs, oc, ph, pw}, x.dtype());
            check(ag_conv2_relu_max_pool2_forward(
                x.device(), x.dtype(), x.data(), bs, ic, ih, iw, w.value.data(), oc,
                has_bias ? b.value.data() : nullptr, &copt, relu ? 1 : 0, pool_window[0],
                pool_window[1], y.data()));
            return Variable{y, nullptr};
        }
        Tensor y = Tensor::uninit(pool, {bs, oc, oh, ow}, x.dtype());
        check(ag_conv2_forward(x.device(), x.dtype(), x.data(), bs, ic, ih, iw, w.value.data(), oc,
                               has_bias ? b.value.data() : nullptr, &copt, relu ? 1 : 0,
                               y.data()));
        return attach(pool, input, y);
    }
    // The layer's output variable around y = conv2(input) (+ bias) that the caller has
    // computed: the backward edges of Conv2::forward.
    Variable attach(Pool &pool, const Variable &input, const Tensor &y) {
        const Tensor &x = input.value;
        const int64_t bs = x.dim(0), ic = x.dim(1), ih = x.dim(2), iw = x.dim(3);
        const int64_t oc = weight.value.dim(0), oh = y.dim(2), ow = y.dim(3);
        const Shape filter = {weight.value.dim(2), weight.value.dim(3)};
        const ag_conv2_options copt = to_c_options(filter, options);
        Variable w = weight.to_variable();
        Variable b = has_bias ? bias.to_variable() : Variable{};
        VariableBuilder builder;
        Pool *pp = &pool;
        if (input.node) {
            Tensor wv = w.value;
            builder.edge(input.node, [=](const Tensor &dy, Tensor *) {
                Tensor dx = Tensor::uninit(*pp, {bs, ic, ih, iw}, dy.dtype());
                check(ag_conv2_backward_input(dy.device(), dy.dtype(), wv.data(), oc, ic, dy.data(),
                                              bs, ih, iw, &copt, dx.data()));
                return dx;
            });
        }
        if (w.node) {
            Tensor xv = x;
            Shape wshape = weight.value.shape();
            builder.edge(w.node, [=](const Tensor &dy, Tensor *into) {
                Tensor dw = into ? *into : Tensor::uninit(*pp, wshape, dy.dtype());
                check(ag_conv2_backward_weight(dy.device(), dy.dtype(), xv.data(), bs, ic, ih, iw,
                                               dy.data(), oc, &copt, 0.f, dw.data()));
                return dw;
            });
        }
        if (b.node) {
            builder.edge(b.node, [=](const Tensor &dy, Tensor *into) {
                Tensor db = into ? *into : Tensor::uninit(*pp, {oc}, dy.dtype());
                check(ag_bias_grad(dy.device(), dy.dtype(), dy.data(), bs, oc, oh * ow, 0.f,
                                   db.data()));
                return db;
            });
        }
        return builder.build(y);
    }
};

// Dense (layer.rs:1070-1143): Y = X.W (+ b), W is [inputs, outputs];
// edges dX = dY.W^T, dW = X^T.dY (Variable2::dot, autograd.rs:607-627),
// db = column sum of dY (broadcast_backward, autograd.rs:490-542).
class Dense : public Layer {
   public:
    Parameter weight;  // [inputs, outputs]
    bool has_bias = false;
    Parameter bias;    // [outputs]
    // A layer that shares the parameters of an earlier Dense (one Parameter used by two
    // layers: its node then receives two gradients, summed in arrival order,
    // autograd.rs:126-131).  The owner's Parameter objects are used; this layer's stay empty.
    Dense *tied = nullptr;
    Shape weight_shape;  // [inputs, outputs], known before the value exists
    Parameter &W() { return tied ? tied->weight : weight; }
    Parameter &B() { return tied ? tied->bias : bias; }
    const Parameter &W() const { return tied ? tied->weight : weight; }
    const Parameter &B() const { return tied ? tied->bias : bias; }

    const char *name() const override { return "Dense"; }
    void parameters(std::vector<Parameter *> &out) override {
        if (tied) return;  // visited through the owner
        out.push_back(&weight);
        if (has_bias) out.push_back(&bias);
    }
    Variable forward(Pool &pool, const Variable &input) override {
        return forward_fused(pool, input, false);
    }
    bool records_gradient(const Variable &input) const {
        return input.node || W().node || (has_bias && B().node);
    }
    // Forward with the bias add (and, when no gradient is recorded, the following
    // Relu) folded into the product's epilogue.
    Variable forward_fused(Pool &pool, const Variable &input, bool relu) {
        const Tensor &x = input.value;
        if (x.ndim() != 2) throw Error(AG_ERR_SHAPE, "Dense needs a 2-D input");
        if (!x.is_standard_layout()) throw Error(AG_ERR_SHAPE, "Dense needs standard layout");
        Variable w = W().to_variable();
        if (x.dim(1) != w.value.dim(0))
            throw Error(AG_ERR_SHAPE, "a_cols != b_rows, " + std::to_string(x.dim(1)) +
                                          " != " + std::to_string(w.value.dim(0)));
        if (relu && records_gradient(input))
            throw Error(AG_ERR_INVALID, "Dense: fused relu while a gradient is recorded");
        const int64_t bs = x.dim(0), ins = x.dim(1), outs = w.value.dim(1);
        Variable b = has_bias ? B().to_variable() : Variable{};
        Tensor y = Tensor::uninit(pool, {bs, outs}, x.dtype());
        check(ag_dense_forward(x.device(), x.dtype(), x.data(), bs, ins, w.value.data(), outs,
                               has_bias ? b.value.data() : nullptr, relu ? 1 : 0, y.data()));
        return attach(pool, input, y);
    }
    // The layer's output variable around y = Dense(input) that the caller has computed:
    // the three backward edges of Dense::forward.
    Variable attach(Pool &pool, const Variable &input, const Tensor &y) {
        const Tensor &x = input.value;
        Variable w = W().to_variable();
        Variable b = has_bias ? B().to_variable() : Variable{};
        const int64_t bs = x.dim(0), outs = w.value.dim(1);
        VariableBuilder builder;
        Pool *pp = &pool;
        if (input.node) {
            Tensor wv = w.value;
            builder.edge(input.node, [=](const Tensor &dy, Tensor *) { return dy.dot(*pp, wv.t()); });
        }
        if (w.node) {
            Tensor xv = x;
            builder.edge(w.node, [=](const Tensor &dy, Tensor *into) {
                if (into) {
                    xv.t().gemm_into(1.f, dy, 0.f, *into);
                    return *into;
                }
                return xv.t().dot(*pp, dy);
            });
        }
        if (has_bias && b.node) {
            builder.edge(b.node, [=](const Tensor &dy, Tensor *into) {
                Tensor db = into ? *into : Tensor::uninit(*pp, {outs}, dy.dtype());
                check(ag_bias_grad(dy.device(), dy.dtype(), dy.data(), bs, outs, 1, 0.f,
                                   db.data()));
                return db;
            });
        }
        return builder.build(y);
    }
};

// MaxPool2 (layer.rs:1193-1216): the backward edge clones the input and runs
// max_pool2_backward in place on the clone.
class MaxPool2 : public Layer {
   public:
    int filter[2] = {2, 2};
    int stride[2] = {2, 2};  // defaults to the filter (layer.rs:535-539)

    const char *name() const override { return "MaxPool2"; }
    Variable forward(Pool &pool, const Variable &input) override {
        const Tensor &x = input.value;
        if (x.ndim() != 4 || !x.is_standard_layout())
            throw Error(AG_ERR_SHAPE, "MaxPool2 needs a standard-layout 4-D input");
        const int64_t bs = x.dim(0), c = x.dim(1), ih = x.dim(2), iw = x.dim(3);
        if (ih < filter[0] || iw < filter[1])
            throw Error(AG_ERR_SHAPE, "MaxPool2: window larger than input");
        const int64_t oh = (ih - filter[0]) / stride[0] + 1, ow = (iw - filter[1]) / stride[1] + 1;
        Tensor y = Tensor::uninit(pool, {bs, c, oh, ow}, x.dtype());
        const int f0 = filter[0], f1 = filter[1], s0 = stride[0], s1 = stride[1];
        check(ag_max_pool2(x.device(), x.dtype(), x.data(), bs, c, ih, iw, f0, f1, s0, s1,
                           y.data()));
        VariableBuilder builder;
        Pool *pp = &pool;
        if (input.node) {
            Tensor xv = x;
            builder.edge(input.node, [=](const Tensor &dy, Tensor *) {
                Tensor dx = Tensor::uninit(*pp, xv.shape(), xv.dtype());
                // clone of the input + in-place backward of the reference, in one pass
                check(ag_max_pool2_backward_from_input(xv.device(), xv.dtype(), xv.data(), bs, c, ih,
                                                       iw, f0, f1, s0, s1, dy.data(), dx.data()));
                return dx;
            });
        }
        return builder.build(y);
    }
};

// Relu (layer.rs:1254-1298): in place when the input buffer is not shared and
// no gradient is needed, else out of place; the backward edge gates on the
// layer input.
class Relu : public Layer {
   public:
    const char *name() const override { return "Relu"; }
    Variable forward(Pool &pool, const Variable &input) override {
        const Tensor &x = input.value;
        if (!x.is_standard_layout()) throw Error(AG_ERR_SHAPE, "Relu needs standard layout");
        Tensor y = (!input.node && x.exclusive()) ? x : Tensor::uninit(pool, x.shape(), x.dtype());
        check(ag_relu(x.device(), x.dtype(), x.data(), y.data(), x.len()));
        return attach(pool, input, y);
    }
    // The output variable around y = relu(input) that the caller has computed.
    static Variable attach(Pool &pool, const Variable &input, const Tensor &y) {
        const Tensor &x = input.value;
        VariableBuilder builder;
        Pool *pp = &pool;
        if (input.node) {
            Tensor xv = x;
            builder.edge(input.node, [=](const Tensor &dy, Tensor *) {
                Tensor dx = dy.exclusive() ? dy : Tensor::uninit(*pp, dy.shape(), dy.dtype());
                check(ag_relu_backward(dy.device(), dy.dtype(), xv.data(), dy.data(), dx.data(),
                                       dy.len()));
                return dx;
            });
        }
        return builder.build(y);
    }
};

// Relu followed by a 2x2 / stride 2 MaxPool2 over even planes as one kernel each way: the
// Relu's output is never stored and the single backward edge produces the gradient at the
// Relu's input (the values are those of the two layers run one after the other).
inline bool relu_pool_fusable(const Variable &input, const MaxPool2 &mp) {
    const Tensor &x = input.value;
    return mp.filter[0] == 2 && mp.filter[1] == 2 && mp.stride[0] == 2 && mp.stride[1] == 2 &&
           x.ndim() == 4 && x.is_standard_layout() && x.dim(2) >= 2 && x.dim(3) >= 2 &&
           x.dim(2) % 2 == 0 && x.dim(3) % 2 == 0;
}
inline Variable relu_pool_attach(Pool &pool, const Variable &input, const Tensor &y);
inline Variable relu_pool_forward(Pool &pool, const Variable &input) {
    const Tensor &x = input.value;
    const int64_t bs = x.dim(0), c = x.dim(1), ih = x.dim(2), iw = x.dim(3);
    Tensor y = Tensor::uninit(pool, {bs, c, ih / 2, iw / 2}, x.dtype());
    check(ag_relu_max_pool2_forward(x.device(), x.dtype(), x.data(), bs, c, ih, iw, y.data()));
    return relu_pool_attach(pool, input, y);
}
// The pooled variable around y = max_pool2(relu(input)) that the caller has computed.
inline Variable relu_pool_attach(Pool &pool, const Variable &input, const Tensor &y) {
    const Tensor &x = input.value;
    const int64_t bs = x.dim(0), c = x.dim(1), ih = x.dim(2), iw = x.dim(3);
    VariableBuilder builder;
    Pool *pp = &pool;
    if (input.node) {
        Tensor xv = x;
        builder.edge(input.node, [=](const Tensor &dy, Tensor *) {
            Tensor dx = Tensor::uninit(*pp, xv.shape(), xv.dtype());
            check(ag_relu_max_pool2_backward(xv.device(), xv.dtype(), xv.data(), bs, c, ih, iw,
                                             dy.data(), dx.data()));
            return dx;
        });
    }
    return builder.build(y);
}

// Conv2 -> Relu -> 2x2 MaxPool2 of a gradient-recording pass in one forward call that keeps
// the convolution's output; the two nodes (convolution, Relu + pool) are those of the
// separate layers.
inline Variable conv_relu_pool_forward(Pool &pool, Conv2 &conv, const Variable &input) {
    const Tensor &x = input.value;
    if (x.ndim() != 4 || x.dim(1) != conv.weight.value.dim(1))
        throw Error(AG_ERR_SHAPE, "Conv2: input channels do not match the weight");
    if (!x.is_standard_layout()) throw Error(AG_ERR_SHAPE, "Conv2 needs standard layout");
    const int64_t bs = x.dim(0), ic = x.dim(1), ih = x.dim(2), iw = x.dim(3);
    const int64_t oc = conv.weight.value.dim(0);
    const Shape filter = {conv.weight.value.dim(2), conv.weight.value.dim(3)};
    const ag_conv2_options copt = to_c_options(filter, conv.options);
    int64_t oh = 0, ow = 0;
    check(ag_conv2_output_shape(ih, iw, &copt, &oh, &ow));
    Tensor pre = Tensor::uninit(pool, {bs, oc, oh, ow}, x.dtype());
    Tensor y = Tensor::uninit(pool, {bs, oc, oh / 2, ow / 2}, x.dtype());
    check(ag_conv2_relu_max_pool2_forward_keep(
        x.device(), x.dtype(), x.data(), bs, ic, ih, iw, conv.weight.value.data(), oc,
        conv.has_bias ? conv.bias.value.data() : nullptr, &copt, pre.data(), y.data()));
    return relu_pool_attach(pool, conv.attach(pool, input, pre), y);
}

// Flatten (layer.rs:1224-1231): reshape to [batch, rest]; the edge reshapes back.
class Flatten : public Layer {
   public:
    const char *name() const override { return "Flatten"; }
    Variable forward(Pool &, const Variable &input) override {
        const Tensor &x = input.value;
        Shape in_shape = x.shape();
        int64_t bs = x.ndim() ? x.dim(0) : 1;
        Tensor y = x.into_shape({bs, bs ? x.len() / bs : 0});
        VariableBuilder builder;
        if (input.node)
            builder.edge(input.node,
                         [=](const Tensor &dy, Tensor *) { return dy.into_shape(in_shape); });
        return builder.build(y);
    }
};

// Variable2::cross_entropy_loss (neural_network/criterion.rs:30-77): the value
// is the summed loss as a host f32; the edge is dx = (dy/bs)(softmax - onehot).
struct Loss {
    float value = 0.f;
    std::shared_ptr<Node> node;
    void backward() {
        if (!node) return;
        // Seed gradient of a scalar loss is one (Node::backward, autograd.rs:224-235).
        Tensor seed;  // not materialised: the only consumer is the loss edge, which uses dy = 1
        backward_from(node, seed);
    }
};

// loss_dev == null: the value is read back (synchronises), as the reference does.
// loss_dev != null: the value is left in device memory and loss.value stays 0, so that
// the whole step can be enqueued without a host round trip.
inline Loss cross_entropy_loss(Pool &pool, const Variable &input, const Tensor &target,
                               float *loss_dev = nullptr) {
    const Tensor &x = input.value;
    if (x.ndim() != 2 || target.ndim() != 1 || target.dim(0) != x.dim(0))
        throw Error(AG_ERR_SHAPE, "Expected target with shape [" + std::to_string(x.dim(0)) + "]");
    Loss loss;
    if (loss_dev && input.node) {
        // The only consumer of this loss's node is Loss::backward with the seed gradient 1:
        // compute the edge's result now, in the kernel that already has every row's sums.
        Tensor dx = Tensor::uninit(pool, x.shape(), x.dtype());
        check(ag_cross_entropy_loss_device_grad(x.device(), x.dtype(), target.dtype(), x.data(),
                                                target.data(), x.dim(0), x.dim(1), loss_dev, 1.f,
                                                dx.data()));
        loss.node = std::make_shared<Node>();
        ++input.node->pending;
        loss.node->edges.push_back(Edge{input.node, [=](const Tensor &, Tensor *) { return dx; }});
        return loss;
    }
    if (loss_dev)
        check(ag_cross_entropy_loss_device(x.device(), x.dtype(), target.dtype(), x.data(),
                                           target.data(), x.dim(0), x.dim(1), loss_dev));
    else
        check(ag_cross_entropy_loss(x.device(), x.dtype(), target.dtype(), x.data(), target.data(),
                                    x.dim(0), x.dim(1), &loss.value));
    if (input.node) {
        Pool *pp = &pool;
        Tensor xv = x, tv = target;
        loss.node = std::make_shared<Node>();
        ++input.node->pending;
        loss.node->edges.push_back(Edge{input.node, [=](const Tensor &, Tensor *) {
            Tensor dx = Tensor::uninit(*pp, xv.shape(), xv.dtype());
            check(ag_cross_entropy_loss_backward(xv.device(), xv.dtype(), tv.dtype(), xv.data(),
                                                 tv.data(), xv.dim(0), xv.dim(1), 1.f, dx.data()));
            return dx;
        }});
    }
    return loss;
}

}  // namespace autograph
