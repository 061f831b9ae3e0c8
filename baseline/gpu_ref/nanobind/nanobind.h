// Stand-in for the nanobind headers, just large enough to compile the reference's
// sphops/sph_cuda.cu without nanobind or Python: the binding block at the end of that file
// (NB_MODULE) becomes an unused static function whose class_/def calls swallow their arguments,
// and nb::ndarray (ndarray.h) is a plain {pointer, shape} view that the driver fills from raw
// device pointers.  Nothing here is nanobind code.
#pragma once
#include <cstddef>
#include <cstdint>
#include <utility>

namespace nanobind {

struct arg {
    constexpr explicit arg(const char *) {}
    template <typename T>
    arg &operator=(T &&) { return *this; }
};

namespace literals {
constexpr arg operator""_a(const char *name, size_t) { return arg(name); }
}  // namespace literals

template <typename... Args>
struct init {};

struct module_ {
    template <typename... A>
    module_ &def(A &&...) { return *this; }
    template <typename... A>
    module_ &attr(A &&...) { return *this; }
    const char *doc() const { return ""; }
};

template <typename T>
struct class_ {
    template <typename... A>
    class_(module_ &, const char *, A &&...) {}
    template <typename... A>
    class_ &def(A &&...) { return *this; }
    template <typename... A>
    class_ &def_prop_ro(A &&...) { return *this; }
    template <typename... A>
    class_ &def_prop_rw(A &&...) { return *this; }
    template <typename... A>
    class_ &def_ro(A &&...) { return *this; }
};

}  // namespace nanobind

#define NB_MODULE(name, variable) [[maybe_unused]] static void nanobind_stub_module_##name(::nanobind::module_ &variable)
