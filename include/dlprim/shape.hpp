// Tensor shape of up to 8 dimensions (the reference's include/dlprim/shape.hpp:25-170).
#pragma once
#include <dlprim/definitions.hpp>
#include <array>
#include <ostream>
#include <vector>

namespace dlprim {

class DLPRIM_API Shape {
public:
    Shape() : dims_{}, size_(0) {}
    Shape(size_t a) : dims_{a}, size_(1) {}
    Shape(size_t a, size_t b) : dims_{a, b}, size_(2) {}
    Shape(size_t a, size_t b, size_t c) : dims_{a, b, c}, size_(3) {}
    Shape(size_t a, size_t b, size_t c, size_t d) : dims_{a, b, c, d}, size_(4) {}
    Shape(size_t a, size_t b, size_t c, size_t d, size_t e) : dims_{a, b, c, d, e}, size_(5) {}

    template<typename It>
    static Shape from_range(It begin, It end)
    {
        Shape s;
        for(; begin != end; ++begin) {
            if(s.size_ >= max_tensor_dim) throw ValidationError("Unsupported tensor size");
            s.dims_[s.size_++] = size_t(*begin);
        }
        return s;
    }
    bool operator==(Shape const &o) const
    {
        if(size_ != o.size_) return false;
        for(int i = 0; i < size_; i++)
            if(dims_[i] != o.dims_[i]) return false;
        return true;
    }
    bool operator!=(Shape const &o) const { return !(*this == o); }
    int size() const { return size_; }
    size_t &operator[](int i) { return dims_[i]; }
    size_t operator[](int i) const { return dims_[i]; }
    size_t total_size() const
    {
        if(size_ == 0) return 0;
        size_t r = 1;
        for(int i = 0; i < size_; i++) r *= dims_[i];
        return r;
    }
    size_t size_no_batch() const
    {
        if(size_ == 0) return 0;
        size_t r = 1;
        for(int i = 1; i < size_; i++) r *= dims_[i];
        return r;
    }
    size_t const *begin() const { return &dims_[0]; }
    size_t const *end() const { return begin() + size_; }
    /// Remove every dimension equal to 1, e.g. (4,5,1,1) -> (4,5).
    Shape squeeze() const
    {
        Shape r;
        for(int i = 0; i < size_; i++)
            if(dims_[i] != 1) r.dims_[r.size_++] = dims_[i];
        return r;
    }
private:
    std::array<size_t, max_tensor_dim> dims_;
    int size_;
};

inline std::ostream &operator<<(std::ostream &o, Shape const &s)
{
    o << '(';
    for(int i = 0; i < s.size(); i++) o << (i ? "," : "") << s[i];
    return o << ')';
}

} // namespace dlprim
