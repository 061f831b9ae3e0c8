// Stand-in for nanobind/ndarray.h: a {pointer, shape} view with the accessors the reference's
// kernels call (data, shape, ndim, size).  See nanobind.h in this directory.
#pragma once
#include <cstddef>
#include <cstdint>
#include <initializer_list>

namespace nanobind {

template <long... Dims>
struct shape {};
struct c_contig {};
namespace device {
struct cuda {};
struct cpu {};
}  // namespace device

template <typename T, typename... Tags>
class ndarray {
public:
    ndarray() = default;
    ndarray(T *data, std::initializer_list<size_t> dims) : data_(data) {
        for (size_t d : dims) shape_[ndim_++] = d;
    }
    T *data() const { return data_; }
    size_t ndim() const { return ndim_; }
    size_t shape(size_t i) const { return shape_[i]; }
    size_t size() const {
        size_t n = 1;
        for (size_t i = 0; i < ndim_; ++i) n *= shape_[i];
        return n;
    }

private:
    T *data_ = nullptr;
    size_t ndim_ = 0;
    size_t shape_[6] = {0, 0, 0, 0, 0, 0};
};

}  // namespace nanobind
