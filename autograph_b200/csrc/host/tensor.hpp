// Host-side tensor over device memory: the counterpart of the reference's
// TensorBase / ScalarTensorBase (src/tensor.rs:327-332, 1256-1261) restricted to
// what the dense-contraction path needs.  A tensor is (shared buffer, dtype,
// shape, element strides, element offset); transposes and reshapes are views,
// never copies (t() = stride swap, src/tensor.rs:1642-1644).
#pragma once

#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/autograph_b200.h"

namespace autograph {

// Error carried across the host layer; converted to an ag_status at the C ABI.
class Error : public std::runtime_error {
   public:
    Error(int status, const std::string &msg) : std::runtime_error(msg), status_(status) {}
    int status() const { return status_; }

   private:
    int status_;
};

inline void check(int status) {
    if (status != AG_OK) throw Error(status, ag_last_error());
}

using Shape = std::vector<int64_t>;

inline int64_t numel(const Shape &s) {
    int64_t n = 1;
    for (int64_t d : s) n *= d;
    return n;
}

inline size_t element_size(ag_dtype t) {
    switch (t) {
        case AG_F32: return 4;
        case AG_BF16: return 2;
        case AG_U8: return 1;
        case AG_U16: return 2;
        case AG_U32: return 4;
    }
    return 0;
}

// Caching device allocator.  Every block is used on one in-order stream, so a
// released block can be handed out again without synchronising: work that
// still reads it was submitted earlier on the same stream.
class Pool {
   public:
    explicit Pool(ag_device *dev) : dev_(dev) {}
    Pool(const Pool &) = delete;
    Pool &operator=(const Pool &) = delete;
    ~Pool() {
        for (auto &kv : free_)
            for (void *p : kv.second) ag_free(dev_, p);
    }
    ag_device *device() const { return dev_; }
    // New tensors are bound to `dev` (another stream of the same GPU) from now on.
    void set_device(ag_device *dev) { dev_ = dev; }
    void *acquire(size_t bytes, size_t *granted) {
        size_t cls = size_class(bytes);
        *granted = cls;
        auto it = free_.find(cls);
        if (it != free_.end() && !it->second.empty()) {
            void *p = it->second.back();
            it->second.pop_back();
            return p;
        }
        void *p = nullptr;
        check(ag_alloc(dev_, cls, &p));
        return p;
    }
    void release(void *p, size_t cls) {
        if (hold_)
            hold_->push_back({p, cls});
        else
            free_[cls].push_back(p);
    }
    // While a sink is set, released blocks are parked in it instead of becoming
    // reusable.  A captured CUDA graph keeps the addresses of its intermediate
    // buffers; parking them keeps those buffers private to the graph.
    using Parked = std::vector<std::pair<void *, size_t>>;
    void set_hold(Parked *sink) { hold_ = sink; }
    void unpark(Parked &blocks) {
        for (auto &b : blocks) free_[b.second].push_back(b.first);
        blocks.clear();
    }

   private:
    static size_t size_class(size_t bytes) {
        size_t c = 512;
        while (c < bytes) c <<= 1;
        // Above 1 MiB round to the next multiple of 1/8 of the power of two below.
        if (c > (size_t(1) << 20)) {
            size_t step = c >> 4;
            size_t r = (bytes + step - 1) / step * step;
            return r;
        }
        return c;
    }
    ag_device *dev_;
    std::map<size_t, std::vector<void *>> free_;
    Parked *hold_ = nullptr;
};

struct Buffer {
    Pool *pool = nullptr;  // null: memory not owned (external pointer)
    void *ptr = nullptr;
    size_t granted = 0;
    ~Buffer() {
        if (pool && ptr) pool->release(ptr, granted);
    }
};

class Tensor {
   public:
    Tensor() = default;

    static Tensor uninit(Pool &pool, const Shape &shape, ag_dtype dtype) {
        Tensor t;
        t.dev_ = pool.device();
        t.dtype_ = dtype;
        t.shape_ = shape;
        t.strides_ = contiguous_strides(shape);
        auto buf = std::make_shared<Buffer>();
        size_t bytes = (size_t)numel(shape) * element_size(dtype);
        buf->ptr = pool.acquire(bytes ? bytes : 1, &buf->granted);
        buf->pool = &pool;
        t.buf_ = std::move(buf);
        return t;
    }
    static Tensor zeros(Pool &pool, const Shape &shape, ag_dtype dtype) {
        Tensor t = uninit(pool, shape, dtype);
        check(ag_fill_zero(t.dev_, t.data(), t.nbytes()));
        return t;
    }
    // ≙ Tensor::from(vec).into_device(device)
    static Tensor from_host(Pool &pool, const Shape &shape, ag_dtype dtype, const void *host) {
        Tensor t = uninit(pool, shape, dtype);
        check(ag_upload(t.dev_, t.data(), host, t.nbytes()));
        return t;
    }
    // View over memory the caller owns (no copy, not freed).
    static Tensor external(ag_device *dev, void *ptr, const Shape &shape, ag_dtype dtype) {
        Tensor t;
        t.dev_ = dev;
        t.dtype_ = dtype;
        t.shape_ = shape;
        t.strides_ = contiguous_strides(shape);
        auto buf = std::make_shared<Buffer>();
        buf->ptr = ptr;
        t.buf_ = std::move(buf);
        return t;
    }

    bool defined() const { return (bool)buf_; }
    ag_device *device() const { return dev_; }
    ag_dtype dtype() const { return dtype_; }
    const Shape &shape() const { return shape_; }
    const Shape &strides() const { return strides_; }
    int64_t dim(size_t i) const { return shape_.at(i); }
    size_t ndim() const { return shape_.size(); }
    int64_t len() const { return numel(shape_); }
    size_t nbytes() const { return (size_t)len() * element_size(dtype_); }
    int64_t offset() const { return offset_; }
    void *base() const { return buf_->ptr; }
    void *data() const { return (char *)buf_->ptr + offset_ * (int64_t)element_size(dtype_); }
    // True when no other tensor shares the buffer (≙ ArcTensor::get_view_mut succeeding).
    bool exclusive() const { return buf_ && buf_.use_count() == 1 && buf_->pool != nullptr; }

    bool is_standard_layout() const { return strides_ == contiguous_strides(shape_); }

    // ≙ t(): swap the two axes of a 2-D view.
    Tensor t() const {
        require(ndim() == 2, "t() needs a 2-D tensor");
        Tensor r = *this;
        std::swap(r.shape_[0], r.shape_[1]);
        std::swap(r.strides_[0], r.strides_[1]);
        return r;
    }
    // ≙ into_shape: only for standard layout, like the reference (src/tensor.rs into_shape).
    Tensor into_shape(const Shape &shape) const {
        require(is_standard_layout(), "into_shape needs standard layout");
        require(numel(shape) == len(), "into_shape: element count differs");
        Tensor r = *this;
        r.shape_ = shape;
        r.strides_ = contiguous_strides(shape);
        return r;
    }
    // Slice [begin, begin+count) of axis 0 of a standard-layout tensor.
    Tensor narrow0(int64_t begin, int64_t count) const {
        require(is_standard_layout() && ndim() >= 1, "narrow0 needs standard layout");
        require(begin >= 0 && begin + count <= shape_[0], "narrow0 out of range");
        Tensor r = *this;
        r.shape_[0] = count;
        r.offset_ = offset_ + begin * strides_[0];
        return r;
    }

    // ≙ Dot for ScalarTensorBase (src/tensor/linalg.rs:425-468): C = A.B into a fresh tensor.
    Tensor dot(Pool &pool, const Tensor &rhs) const {
        if (dtype_ != rhs.dtype_)
            throw Error(AG_ERR_DTYPE, "Can not dot tensors of different types");
        require(ndim() == 2 && rhs.ndim() == 2, "dot needs 2-D tensors");
        if (shape_[1] != rhs.shape_[0])
            throw Error(AG_ERR_SHAPE, "a_cols != b_rows, " + std::to_string(shape_[1]) +
                                          " != " + std::to_string(rhs.shape_[0]));
        Tensor out = uninit(pool, {shape_[0], rhs.shape_[1]}, dtype_);
        gemm_into(1.f, rhs, 0.f, out);
        return out;
    }
    // out = alpha * this . rhs + beta * out (≙ fn gemm, src/tensor/linalg.rs:249-360).
    void gemm_into(float alpha, const Tensor &rhs, float beta, Tensor &out) const {
        check(ag_gemm(dev_, dtype_, shape_[0], shape_[1], rhs.shape_[1], alpha, base(), offset_,
                      strides_[0], strides_[1], rhs.base(), rhs.offset_, rhs.strides_[0],
                      rhs.strides_[1], beta, out.base(), out.offset_, out.strides_[0],
                      out.strides_[1]));
    }
    // ≙ scaled_add (src/tensor/ops.rs:257-318), standard layout only.
    void scaled_add(float alpha, const Tensor &x) {
        require(is_standard_layout() && x.is_standard_layout() && x.len() == len() &&
                    x.dtype_ == dtype_,
                "scaled_add needs matching standard-layout tensors");
        check(ag_scaled_add(dev_, dtype_, alpha, x.data(), data(), len()));
    }
    // ≙ into_array (blocking device -> host copy), standard layout only.
    void to_host(void *dst) const {
        require(is_standard_layout(), "to_host needs standard layout");
        check(ag_download(dev_, dst, data(), nbytes()));
    }

    static Shape contiguous_strides(const Shape &shape) {
        Shape s(shape.size());
        int64_t acc = 1;
        for (size_t i = shape.size(); i-- > 0;) {
            s[i] = acc;
            acc *= shape[i];
        }
        return s;
    }

   private:
    static void require(bool ok, const char *msg) {
        if (!ok) throw Error(AG_ERR_SHAPE, msg);
    }
    ag_device *dev_ = nullptr;
    ag_dtype dtype_ = AG_F32;
    Shape shape_, strides_;
    int64_t offset_ = 0;
    std::shared_ptr<Buffer> buf_;
};

}  // namespace autograph
