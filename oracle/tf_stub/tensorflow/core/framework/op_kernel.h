// TEST INFRASTRUCTURE ONLY.
//
// A minimal stand-in for TensorFlow's "tensorflow/core/framework/op_kernel.h",
// just large enough that the CPU kernels of the HGCalML custom ops
// (modules/compiled/*_kernel.cc) compile unmodified WITHOUT TensorFlow.  It is
// used only to build the checker library of the test suite; nothing that
// ships links against it.  The OpKernel classes in those files are compiled
// but never instantiated: the glue code calls the functors directly.
//
// GOOGLE_CUDA must stay undefined so only the CPU specialisations are built.
#ifndef HGC_ORACLE_TF_STUB_OP_KERNEL_H
#define HGC_ORACLE_TF_STUB_OP_KERNEL_H

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstddef>
#include <initializer_list>
#include <stdexcept>
#include <string>
#include <vector>

namespace Eigen {
struct ThreadPoolDevice {};
struct GpuDevice {};
}  // namespace Eigen

namespace tensorflow {

struct Status {
    bool ok_ = true;
    bool ok() const { return ok_; }
};

namespace errors {
template <typename... A>
inline Status InvalidArgument(A...) { Status s; s.ok_ = false; return s; }
}  // namespace errors

enum DataType { DT_INT32, DT_FLOAT };

class TensorShape {
public:
    TensorShape() {}
    TensorShape(std::initializer_list<long long> d) : dims_(d) {}
    void AddDim(long long d) { dims_.push_back(d); }
    std::vector<long long> dims_;
};

template <typename T>
struct FlatView {
    T *p;
    T *data() const { return p; }
};

class Tensor {
public:
    long long dim_size(int i) const { return shape_.dims_.at(i); }
    long long NumElements() const {
        long long n = 1;
        for (auto d : shape_.dims_) n *= d;
        return n;
    }
    const TensorShape &shape() const { return shape_; }
    template <typename T> FlatView<T> flat() { return FlatView<T>{(T *)buf_}; }
    template <typename T> FlatView<const T> flat() const { return FlatView<const T>{(const T *)buf_}; }
    TensorShape shape_;
    void *buf_ = nullptr;
};

class OpKernelConstruction {
public:
    template <typename T> Status GetAttr(const char *, T *) { return Status(); }
};

class OpKernelContext {
public:
    const Tensor &input(int) { static Tensor t; return t; }
    Status allocate_output(int, const TensorShape &, Tensor **) { return Status(); }
    Status allocate_temp(DataType, const TensorShape &, Tensor *) { return Status(); }
    template <typename D> const D &eigen_device() { static D d; return d; }
};

class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction *) {}
    virtual ~OpKernel() {}
    virtual void Compute(OpKernelContext *) = 0;
};

}  // namespace tensorflow

#define OP_REQUIRES_OK(ctx, expr) do { if (!(expr).ok()) return; } while (0)
#define OP_REQUIRES(ctx, cond, status) do { if (!(cond)) { (void)(status); return; } } while (0)
#define HGC_STUB_CAT_(a, b) a##b
#define HGC_STUB_CAT(a, b) HGC_STUB_CAT_(a, b)
#define REGISTER_KERNEL_BUILDER(...) static int HGC_STUB_CAT(hgc_stub_reg_, __COUNTER__) __attribute__((unused)) = 0

#endif
