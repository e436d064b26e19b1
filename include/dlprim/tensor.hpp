// Tensor: a cheap, reference-counted handle to device memory plus an element offset, with a host
// mirror allocated on first use -- the reference's Tensor (include/dlprim/tensor.hpp:106-294) with
// cl::Buffer replaced by a device pointer.
#pragma once
#include <dlprim/context.hpp>
#include <dlprim/shape.hpp>
#include <memory>

namespace dlprim {

class DLPRIM_API TensorSpecs {
public:
    TensorSpecs(Shape const &s = Shape(), DataType d = float_data, bool trainable = true) : shape_(s), dtype_(d)
    {
        is_trainable_ = trainable && is_floating_point_data_type(d);
    }
    bool operator==(TensorSpecs const &o) const { return shape_ == o.shape_ && dtype_ == o.dtype_ && is_trainable_ == o.is_trainable_; }
    bool operator!=(TensorSpecs const &o) const { return !(*this == o); }
    Shape const &shape() const { return shape_; }
    void shape(Shape const &s) { shape_ = s; }
    DataType dtype() const { return dtype_; }
    bool is_trainable() const { return is_trainable_; }
    void freeze() { is_trainable_ = false; }
    size_t memory_size() const { return shape_.total_size() * size_of_data_type(dtype_); }
private:
    friend class Tensor;
    Shape shape_;
    DataType dtype_;
    bool is_trainable_;
};

class DLPRIM_API Tensor {
public:
    Tensor();
    /// Allocate device memory for the shape.
    Tensor(Context &ctx, Shape const &s, DataType d = float_data, bool is_trainable = true);
    /// Wrap memory owned by the caller (not freed): the counterpart of the reference's
    /// Tensor(cl::Buffer const &, offset, shape) constructor.
    Tensor(void *device_ptr, size_t offset_elements, Shape const &s, DataType d = float_data, bool is_trainable = true);

    TensorSpecs const &specs() const { return *specs_; }
    Shape const &shape() const { return specs_->shape(); }
    DataType dtype() const { return specs_->dtype(); }
    bool is_trainable() const { return specs_->is_trainable(); }
    size_t memory_size() const { return shape().total_size() * size_of_data_type(dtype()); }
    /// Change the shape; the new shape must fit the allocation.
    void reshape(Shape const &ns);

    /// Base of the underlying allocation and the tensor's element offset in it (the pair the
    /// reference hands to kernels as cl::Buffer + offset).
    void *device_buffer() const { return base_; }
    size_t device_offset() const { return offset_; }
    /// Device address of element 0 of this tensor.
    void *device_ptr() const { return static_cast<char *>(base_) + offset_ * size_of_data_type(dtype()); }
    template<typename T> T *device_data() const
    {
        DLPRIM_CHECK(TypeTraits<T>::data_type == dtype());
        return static_cast<T *>(device_ptr());
    }
    /// Pinned host mirror, allocated on first use.
    void *host_data();
    template<typename T> T *data()
    {
        DLPRIM_CHECK(TypeTraits<T>::data_type == dtype());
        return static_cast<T *>(host_data());
    }

    Tensor sub_tensor(size_t offset, Shape const &s, DataType d = float_data, bool trainable = true) const;
    Tensor workspace_as_type(DataType d = float_data) const
    {
        return sub_tensor(0, Shape(memory_size() / size_of_data_type(d)), d);
    }
    Tensor alias() const { return sub_tensor(0, shape(), dtype(), is_trainable()); }
    Tensor alias(Shape const &new_shape) const
    {
        Tensor t = alias();
        t.reshape(new_shape);
        return t;
    }

    void to_device(ExecutionContext const &c, void *host_memory, bool sync = true);
    void to_host(ExecutionContext const &c, void *host_memory, bool sync = true);
    void to_device(ExecutionContext const &c, bool sync = true);
    void to_host(ExecutionContext const &c, bool sync = true);

private:
    struct DeviceMem;
    struct HostMem;
    std::shared_ptr<TensorSpecs> specs_;
    std::shared_ptr<DeviceMem> mem_;
    std::shared_ptr<HostMem> host_;
    void *base_ = nullptr;
    size_t offset_ = 0;       // elements of dtype
    size_t capacity_ = 0;     // bytes available from device_ptr()
};

inline std::ostream &operator<<(std::ostream &out, TensorSpecs const &ts)
{
    return out << '[' << ts.shape() << ",dtype=" << data_type_to_string(ts.dtype()) << ']';
}

} // namespace dlprim
