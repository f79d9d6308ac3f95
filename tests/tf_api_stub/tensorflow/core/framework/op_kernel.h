// TEST INFRASTRUCTURE ONLY: declarations of the small part of TensorFlow's custom-op API that the
// shims in hgcalml_b200/tf_shims use, so that they can be syntax- and type-checked where TensorFlow
// is not installed (tests/test_capi_cpu.py).  Nothing here is functional.
#pragma once
#include <cstdint>
#include <initializer_list>
#include <string>
#include <cuda_runtime.h>

namespace Eigen {
struct GpuDevice { cudaStream_t stream() const; };
struct ThreadPoolDevice {};
}  // namespace Eigen

namespace tensorflow {
typedef unsigned char uint8;
struct Status { bool ok() const; };
Status OkStatus();
namespace errors {
template <typename... A> Status InvalidArgument(A...);
template <typename... A> Status Internal(A...);
}  // namespace errors
enum DataType { DT_INT32, DT_FLOAT, DT_UINT8 };
class TensorShape {
public:
    TensorShape();
    TensorShape(std::initializer_list<int64_t>);
    void AddDim(int64_t);
};
template <typename T> struct Flat { T *data() const; T &operator()(int64_t) const; };
class Tensor {
public:
    int64_t dim_size(int) const;
    int64_t NumElements() const;
    const TensorShape &shape() const;
    template <typename T> Flat<T> flat();
    template <typename T> Flat<const T> flat() const;
};
class OpKernelConstruction {
public:
    template <typename T> Status GetAttr(const char *, T *);
    void SetStatus(const Status &);
};
class OpKernelContext {
public:
    const Tensor &input(int);
    Status allocate_output(int, const TensorShape &, Tensor **);
    Status allocate_temp(DataType, const TensorShape &, Tensor *);
    template <typename D> const D &eigen_device();
    void SetStatus(const Status &);
};
class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction *);
    virtual ~OpKernel();
    virtual void Compute(OpKernelContext *) = 0;
};
struct KernelDefBuilder {
    KernelDefBuilder &Device(const char *);
    KernelDefBuilder &HostMemory(const char *);
};
KernelDefBuilder Name(const char *);
extern const char *const DEVICE_GPU;
extern const char *const DEVICE_CPU;
struct OpDefBuilderStub {
    OpDefBuilderStub &Attr(const char *);
    OpDefBuilderStub &Input(const char *);
    OpDefBuilderStub &Output(const char *);
};
OpDefBuilderStub RegisterOpStub(const char *);
}  // namespace tensorflow

#define HGC_TFSTUB_CAT_(a, b) a##b
#define HGC_TFSTUB_CAT(a, b) HGC_TFSTUB_CAT_(a, b)
#define OP_REQUIRES_OK(ctx, expr) do { ::tensorflow::Status s_ = (expr); if (!s_.ok()) { (ctx)->SetStatus(s_); return; } } while (0)
#define OP_REQUIRES(ctx, cond, status) do { if (!(cond)) { (ctx)->SetStatus(status); return; } } while (0)
#define TF_RETURN_IF_ERROR(expr) do { ::tensorflow::Status s_ = (expr); if (!s_.ok()) return s_; } while (0)
#define REGISTER_OP(name) static ::tensorflow::OpDefBuilderStub HGC_TFSTUB_CAT(hgc_op_, __COUNTER__) = ::tensorflow::RegisterOpStub(name)
#define REGISTER_KERNEL_BUILDER(def, cls) static cls *HGC_TFSTUB_CAT(hgc_kernel_, __COUNTER__)(::tensorflow::OpKernelConstruction *c) { (void)(def); return new cls(c); }
