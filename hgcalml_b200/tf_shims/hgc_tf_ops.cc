// TensorFlow custom-op shims: the registered ops of HGCalML's GravNet / object-condensation
// inference path, forwarding to the C ABI of libhgcalml_b200.so.
//
// Each shim keeps the reference's op name, attributes, input/output order and dtypes
// (modules/compiled/{bin_by_coordinates,binned_select_knn,index_replacer,accumulate_knn,
// accumulate_knn_grad,select_knn_grad,local_distance,push_knn,binned_assign_to_condensates}_module.cc), so the unchanged Python wrappers load it with
// tf.load_op_library.  A shim does shape checks, allocate_output / allocate_temp, and ONE call
// into the library on the op's own CUDA stream; it never synchronises the device.
//
// Written against the C++ op API of TensorFlow 2.10 - 2.15 (OkStatus(), OpKernelContext::allocate_temp
// with a TensorShape, Tensor::flat<T>(), eigen_device<GPUDevice>().stream()); for 2.4 - 2.9 the one
// difference, Status::OK() in place of OkStatus(), is selected from the version header below.
//
// Build (needs a TensorFlow installation):
//   g++ -std=c++17 -shared -fPIC hgc_tf_ops.cc -o hgc_tf_ops.so \
//       $(python -c 'import tensorflow as tf; print(" ".join(tf.sysconfig.get_compile_flags()))') \
//       -I../../include -L.. -lhgcalml_b200 \
//       $(python -c 'import tensorflow as tf; print(" ".join(tf.sysconfig.get_link_flags()))')
#define EIGEN_USE_GPU
#include "tensorflow/core/framework/op.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/shape_inference.h"
#include "tensorflow/core/public/version.h"

#include "hgcalml_b200.h"

namespace tensorflow {
namespace {

typedef Eigen::GpuDevice GPUDevice;

inline hgc_stream_t StreamOf(OpKernelContext *ctx) {
    return static_cast<hgc_stream_t>(ctx->eigen_device<GPUDevice>().stream());
}

#if TF_MAJOR_VERSION < 2 || (TF_MAJOR_VERSION == 2 && TF_MINOR_VERSION < 10)
inline Status OkStatus() { return Status::OK(); }
#endif

inline Status FromHgc(int rc, const char *op) {
    if (rc == HGC_OK) return OkStatus();
    if (rc == HGC_ERR_INVALID_ARGUMENT || rc == HGC_ERR_UNSUPPORTED)
        return errors::InvalidArgument(op, ": ", hgc_strerror(rc));
    return errors::Internal(op, ": ", hgc_strerror(rc), " ", hgc_last_cuda_error());
}

// Scratch memory comes from TensorFlow's allocator (uint8 temp tensor; TF aligns to 64 bytes, the
// library wants 256, so over-allocate and round the pointer up).
struct Workspace {
    Tensor t;
    void *ptr = nullptr;
    size_t bytes = 0;
    Status Allocate(OpKernelContext *ctx, size_t need) {
        TF_RETURN_IF_ERROR(ctx->allocate_temp(DT_UINT8, TensorShape({(int64_t)need + 256}), &t));
        uintptr_t p = reinterpret_cast<uintptr_t>(t.flat<uint8>().data());
        ptr = reinterpret_cast<void *>((p + 255) / 256 * 256);
        bytes = need;
        return OkStatus();
    }
};

// ------------------------------------------------------------------ BinByCoordinates
// nbins (and bin_width) are pinned to host memory: the third output is sized from nbins, which the
// reference reads back with a blocking cudaMemcpy (bin_by_coordinates_kernel.cu.cc:28-34).
class BinByCoordinatesGpuOp : public OpKernel {
public:
    explicit BinByCoordinatesGpuOp(OpKernelConstruction *c) : OpKernel(c) {
        OP_REQUIRES_OK(c, c->GetAttr("calc_n_per_bin", &calc_n_per_bin_));
    }
    void Compute(OpKernelContext *ctx) override {
        const Tensor &coords = ctx->input(0), &rs = ctx->input(1), &bw = ctx->input(2), &nbins = ctx->input(3);
        const int n_vert = coords.dim_size(0), n_coords = coords.dim_size(1), n_rs = rs.dim_size(0);
        OP_REQUIRES(ctx, bw.dim_size(0) == 1,
                    errors::InvalidArgument("BinByCoordinatesOp expects singleton (dim: 1) for bin width."));
        OP_REQUIRES(ctx, nbins.dim_size(0) == n_coords,
                    errors::InvalidArgument("BinByCoordinatesOp expects coordinate dimension for number of bins."));
        int total = n_rs - 1;
        for (int i = 0; i < n_coords; i++) total *= nbins.flat<int>()(i);  // host memory
        Tensor *assigned, *flat, *nper;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, n_coords + 1}, &assigned));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n_vert}, &flat));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(2, {total}, &nper));
        // the kernels read nbins / bin_width on the device: stage the few host values in a temp
        Tensor dev_params;
        OP_REQUIRES_OK(ctx, ctx->allocate_temp(DT_INT32, TensorShape({(int64_t)n_coords + 1}), &dev_params));
        int *d_nbins = dev_params.flat<int>().data();
        float *d_bw = reinterpret_cast<float *>(d_nbins + n_coords);
        auto stream = ctx->eigen_device<GPUDevice>().stream();
        cudaMemcpyAsync(d_nbins, nbins.flat<int>().data(), sizeof(int) * n_coords, cudaMemcpyHostToDevice, stream);
        cudaMemcpyAsync(d_bw, bw.flat<float>().data(), sizeof(float), cudaMemcpyHostToDevice, stream);
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_bin_by_coordinates_workspace_bytes(n_vert, n_coords, n_rs, total)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_bin_by_coordinates(
            coords.flat<float>().data(), rs.flat<int>().data(), d_bw, d_nbins,
            assigned->flat<int>().data(), flat->flat<int>().data(), nper->flat<int>().data(),
            n_vert, n_coords, n_rs, total, calc_n_per_bin_, ws.ptr, ws.bytes, StreamOf(ctx)), "BinByCoordinates"));
    }
private:
    bool calc_n_per_bin_;
};

// ------------------------------------------------------------------ BinnedSelectKnn
class BinnedSelectKnnGpuOp : public OpKernel {
public:
    explicit BinnedSelectKnnGpuOp(OpKernelConstruction *c) : OpKernel(c) {
        OP_REQUIRES_OK(c, c->GetAttr("n_neighbours", &K_));
        OP_REQUIRES_OK(c, c->GetAttr("tf_compatible", &tf_compat_));
        OP_REQUIRES_OK(c, c->GetAttr("use_direction", &use_direction_));
    }
    void Compute(OpKernelContext *ctx) override {
        const Tensor &coords = ctx->input(0), &bin_idx = ctx->input(1), &dim_bin_idx = ctx->input(2),
                     &bounds = ctx->input(3), &n_bins = ctx->input(4), &bw = ctx->input(5), &dir = ctx->input(6);
        const int n_vert = coords.dim_size(0), n_coords = coords.dim_size(1);
        const int n_bb = bounds.dim_size(0), n_bin_dims = n_bins.dim_size(0);
        OP_REQUIRES(ctx, n_bin_dims > 1, errors::InvalidArgument("BinnedSelectKnnOp expects at least 2 binning dimensions."));
        OP_REQUIRES(ctx, n_bin_dims < 6, errors::InvalidArgument("BinnedSelectKnnOp expects maximum 5 binning dimensions."));
        OP_REQUIRES(ctx, dim_bin_idx.dim_size(1) - 1 == n_bin_dims,
                    errors::InvalidArgument("BinnedSelectKnnOp expects number of bin dimensions (including row splits) -1 == number of total bin dimensions."));
        OP_REQUIRES(ctx, n_coords > 1, errors::InvalidArgument("BinnedSelectKnnOp expects at least 2 dimensions."));
        OP_REQUIRES(ctx, n_vert == bin_idx.dim_size(0),
                    errors::InvalidArgument("BinnedSelectKnnOp expects same first dimension for bin idx and coordinates."));
        OP_REQUIRES(ctx, bw.dim_size(0) == 1, errors::InvalidArgument("BinnedSelectKnnOp expects singleton (dim(1)) for bin width."));
        if (use_direction_)
            OP_REQUIRES(ctx, dir.dim_size(0) == n_vert,
                        errors::InvalidArgument("BinnedSelectKnnOp needs a direction tensor with length nvert if use_direction=True."));
        Tensor *idx, *dist;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, K_}, &idx));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n_vert, K_}, &dist));
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_binned_select_knn_workspace_bytes(n_vert, K_, n_coords, n_bin_dims)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_binned_select_knn(
            coords.flat<float>().data(), bin_idx.flat<int>().data(), dir.flat<int>().data(),
            dim_bin_idx.flat<int>().data(), bounds.flat<int>().data(), n_bins.flat<int>().data(),
            bw.flat<float>().data(), idx->flat<int>().data(), dist->flat<float>().data(),
            n_vert, K_, n_coords, n_bin_dims, n_bb, tf_compat_, use_direction_, ws.ptr, ws.bytes, StreamOf(ctx)),
            "BinnedSelectKnn"));
    }
private:
    int K_;
    bool tf_compat_, use_direction_;
};

// ------------------------------------------------------------------ IndexReplacer
class IndexReplacerGpuOp : public OpKernel {
public:
    explicit IndexReplacerGpuOp(OpKernelConstruction *c) : OpKernel(c) {}
    void Compute(OpKernelContext *ctx) override {
        const Tensor &tbr = ctx->input(0), &rep = ctx->input(1);
        Tensor *out;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, tbr.shape(), &out));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_index_replacer(tbr.flat<int>().data(), rep.flat<int>().data(),
                                                       out->flat<int>().data(), tbr.NumElements(), rep.dim_size(0),
                                                       nullptr, StreamOf(ctx)), "IndexReplacer"));
    }
};

// ------------------------------------------------------------------ AccumulateKnn
class AccumulateKnnGpuOp : public OpKernel {
public:
    explicit AccumulateKnnGpuOp(OpKernelConstruction *c) : OpKernel(c) {
        OP_REQUIRES_OK(c, c->GetAttr("n_moments", &n_moments_));
        OP_REQUIRES_OK(c, c->GetAttr("mean_and_max", &mean_and_max_));
    }
    void Compute(OpKernelContext *ctx) override {
        const Tensor &w = ctx->input(0), &feat = ctx->input(1), &idx = ctx->input(2);
        const int n_vert = w.dim_size(0), K = idx.dim_size(1), F = feat.dim_size(1);
        OP_REQUIRES(ctx, n_vert == idx.dim_size(0) && n_vert == feat.dim_size(0),
                    errors::InvalidArgument("AccumulateKnnOp expects first dimensions of all inputs to match."));
        OP_REQUIRES(ctx, K == w.dim_size(1),
                    errors::InvalidArgument("AccumulateKnnOp expects second dimension of distance and neighbour index tensor to match"));
        const int n_out = mean_and_max_ ? 2 * F : F;
        Tensor *out, *maxidx;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, n_out}, &out));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n_vert, F}, &maxidx));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_accumulate_knn(
            w.flat<float>().data(), feat.flat<float>().data(), idx.flat<int>().data(),
            out->flat<float>().data(), maxidx->flat<int>().data(), n_vert, K, F, n_out, n_moments_,
            mean_and_max_, StreamOf(ctx)), "AccumulateKnn"));
    }
private:
    int n_moments_;
    bool mean_and_max_;
};

// ------------------------------------------------------------------ AccumulateKnnGrad
class AccumulateKnnGradGpuOp : public OpKernel {
public:
    explicit AccumulateKnnGradGpuOp(OpKernelConstruction *c) : OpKernel(c) {}
    void Compute(OpKernelContext *ctx) override {
        const Tensor &g = ctx->input(0), &w = ctx->input(1), &feat = ctx->input(2), &idx = ctx->input(3),
                     &maxidx = ctx->input(4);
        const int n_vert = g.dim_size(0), G = g.dim_size(1), K = idx.dim_size(1), F = feat.dim_size(1);
        const bool mean_and_max = G > F;  // detected as in accumulate_knn_grad_kernel.cc:246
        Tensor *gw, *gf;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, K}, &gw));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n_vert, F}, &gf));
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_knn_grad_workspace_bytes(n_vert, K)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_accumulate_knn_grad(
            g.flat<float>().data(), w.flat<float>().data(), feat.flat<float>().data(), maxidx.flat<int>().data(),
            idx.flat<int>().data(), gw->flat<float>().data(), gf->flat<float>().data(), n_vert, K, F, G, 0,
            mean_and_max, ws.ptr, ws.bytes, StreamOf(ctx)), "AccumulateKnnGrad"));
    }
};

// ------------------------------------------------------------------ SelectKnnGrad
class SelectKnnGradGpuOp : public OpKernel {
public:
    explicit SelectKnnGradGpuOp(OpKernelConstruction *c) : OpKernel(c) {}
    void Compute(OpKernelContext *ctx) override {
        const Tensor &g = ctx->input(0), &idx = ctx->input(1), &dist = ctx->input(2), &coord = ctx->input(3);
        const int n_vert = coord.dim_size(0), C = coord.dim_size(1), K = dist.dim_size(1);
        Tensor *out;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, C}, &out));
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_knn_grad_workspace_bytes(n_vert, K)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_select_knn_grad(
            g.flat<float>().data(), idx.flat<int>().data(), dist.flat<float>().data(), coord.flat<float>().data(),
            out->flat<float>().data(), n_vert, K, C, ws.ptr, ws.bytes, StreamOf(ctx)), "SelectKnnGrad"));
    }
};

// ------------------------------------------------------------------ LocalDistance, PushKnn
class LocalDistanceGpuOp : public OpKernel {
public:
    explicit LocalDistanceGpuOp(OpKernelConstruction *c) : OpKernel(c) {}
    void Compute(OpKernelContext *ctx) override {
        const Tensor &coords = ctx->input(0), &idx = ctx->input(1);
        const int n_in = coords.dim_size(0), C = coords.dim_size(1), n_out = idx.dim_size(0), K = idx.dim_size(1);
        Tensor *dist;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_out, K}, &dist));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_local_distance(idx.flat<int>().data(), coords.flat<float>().data(),
                                                       dist->flat<float>().data(), C, n_in, n_out, K, StreamOf(ctx)),
                                    "LocalDistance"));
    }
};

class PushKnnGpuOp : public OpKernel {
public:
    explicit PushKnnGpuOp(OpKernelConstruction *c) : OpKernel(c) {}
    void Compute(OpKernelContext *ctx) override {
        const Tensor &w = ctx->input(0), &feat = ctx->input(1), &idx = ctx->input(2);
        const int n_vert = feat.dim_size(0), F = feat.dim_size(1), K = idx.dim_size(1);
        Tensor *out;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, F}, &out));
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_knn_grad_workspace_bytes(n_vert, K)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_push_knn(w.flat<float>().data(), feat.flat<float>().data(),
                                                 idx.flat<int>().data(), out->flat<float>().data(), n_vert, K, F,
                                                 ws.ptr, ws.bytes, StreamOf(ctx)), "PushKnn"));
    }
};

// ------------------------------------------------------------------ BinnedAssignToCondensates
// The reference registers a CPU kernel only and its wrapper pins the op to '/cpu'
// (modules/assign_condensate_op.py:299); this GPU kernel is picked once that pin is removed.
class BinnedAssignToCondensatesGpuOp : public OpKernel {
public:
    explicit BinnedAssignToCondensatesGpuOp(OpKernelConstruction *c) : OpKernel(c) {
        OP_REQUIRES_OK(c, c->GetAttr("beta_threshold", &beta_threshold_));
        OP_REQUIRES_OK(c, c->GetAttr("assign_by_max_beta", &assign_by_max_beta_));
    }
    void Compute(OpKernelContext *ctx) override {
        const Tensor &cc = ctx->input(0), &dist = ctx->input(1), &mask = ctx->input(3), &bin_splits = ctx->input(5),
                     &itf = ctx->input(6), &orig = ctx->input(7), &rs = ctx->input(8), &n_bins = ctx->input(9),
                     &bw = ctx->input(10), &cc_h = ctx->input(11), &dist_h = ctx->input(12), &beta_h = ctx->input(13),
                     &mask_h = ctx->input(14), &rs_h = ctx->input(15);
        const int n = cc.dim_size(0), n_h = beta_h.dim_size(0), dims = cc.dim_size(1);
        const int dims_binning = n_bins.dim_size(0), num_rows = rs.dim_size(0) - 1;
        Tensor *assigned_h, *assigned, *alpha, *asso, *ncond;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_h}, &assigned_h));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n}, &assigned));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(2, {n_h}, &alpha));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(3, {n}, &asso));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(4, {num_rows + 1}, &ncond));
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_binned_assign_to_condensates_workspace_bytes(n, n_h, num_rows, dims)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_binned_assign_to_condensates(
            dims, dims_binning, cc_h.flat<float>().data(), dist_h.flat<float>().data(), beta_h.flat<float>().data(),
            mask_h.flat<int>().data(), assigned_h->flat<int>().data(), orig.flat<int>().data(),
            rs_h.flat<int>().data(), cc.flat<float>().data(), dist.flat<float>().data(), mask.flat<int>().data(),
            itf.flat<int>().data(), assigned->flat<int>().data(), asso->flat<int>().data(),
            ncond->flat<int>().data(), alpha->flat<int>().data(), bin_splits.flat<int>().data(),
            n_bins.flat<int>().data(), bw.flat<float>().data(), rs.flat<int>().data(), num_rows, n, n_h,
            assign_by_max_beta_, ws.ptr, ws.bytes, StreamOf(ctx)), "BinnedAssignToCondensates"));
    }
private:
    float beta_threshold_;
    bool assign_by_max_beta_;
};

// ------------------------------------------------------------------ wrapper-level ops
// These have no counterpart among the reference's registered ops: each replaces the TensorFlow glue
// of a Python wrapper together with the op inside it, so the wrapper shrinks to one op call.

// BinnedSelectKnn of modules/binned_select_knn_op.py:32-95 (binning, argsort, gathers, the op,
// IndexReplacer, scatter back) in one enqueue.  n_bins <= 0 selects the wrapper's default.
class HgcBinnedSelectKnnRaggedGpuOp : public OpKernel {
public:
    explicit HgcBinnedSelectKnnRaggedGpuOp(OpKernelConstruction *c) : OpKernel(c) {
        OP_REQUIRES_OK(c, c->GetAttr("n_neighbours", &K_));
        OP_REQUIRES_OK(c, c->GetAttr("n_bins", &n_bins_));
        OP_REQUIRES_OK(c, c->GetAttr("max_bin_dims", &max_bin_dims_));
        OP_REQUIRES_OK(c, c->GetAttr("tf_compatible", &tf_compat_));
        OP_REQUIRES_OK(c, c->GetAttr("use_direction", &use_direction_));
    }
    void Compute(OpKernelContext *ctx) override {
        const Tensor &coords = ctx->input(0), &rs = ctx->input(1), &dir = ctx->input(2);
        const int n_vert = coords.dim_size(0), n_coords = coords.dim_size(1), n_rs = rs.dim_size(0);
        Tensor *idx, *dist, *sorting;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, K_}, &idx));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n_vert, K_}, &dist));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(2, {n_vert}, &sorting));
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_binned_select_knn_ragged_workspace_bytes(
                                                 n_vert, K_, n_coords, n_rs, n_bins_, max_bin_dims_)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_binned_select_knn_ragged(
            coords.flat<float>().data(), rs.flat<int>().data(), use_direction_ ? dir.flat<int>().data() : nullptr,
            idx->flat<int>().data(), dist->flat<float>().data(), sorting->flat<int>().data(), n_vert, K_,
            n_coords, n_rs, n_bins_, max_bin_dims_, tf_compat_, use_direction_, ws.ptr, ws.bytes, StreamOf(ctx)),
            "HgcBinnedSelectKnnRagged"));
    }
private:
    int K_, n_bins_, max_bin_dims_;
    bool tf_compat_, use_direction_;
};

// The collection step of RaggedGravNet / DistanceWeightedMessagePassing
// (modules/GravNetLayersRagged.py:3195-3204, 3587-3600): output [N, 2F] = [mean - own | max - own] of
// AccumulateKnn(distance_scale * distsq, features, indices) over the slots first_slot.. of the rows.
class HgcGravnetCollectGpuOp : public OpKernel {
public:
    explicit HgcGravnetCollectGpuOp(OpKernelConstruction *c) : OpKernel(c) {
        OP_REQUIRES_OK(c, c->GetAttr("first_slot", &first_slot_));
        OP_REQUIRES_OK(c, c->GetAttr("distance_scale", &scale_));
        OP_REQUIRES_OK(c, c->GetAttr("subtract_self", &subtract_self_));
    }
    void Compute(OpKernelContext *ctx) override {
        const Tensor &dist = ctx->input(0), &feat = ctx->input(1), &idx = ctx->input(2), &order = ctx->input(3);
        const int n_vert = feat.dim_size(0), F = feat.dim_size(1), ld = idx.dim_size(1);
        OP_REQUIRES(ctx, dist.dim_size(0) == n_vert && idx.dim_size(0) == n_vert && dist.dim_size(1) == ld,
                    errors::InvalidArgument("HgcGravnetCollect expects matching first dimensions and neighbour counts."));
        // order: the sorting output of HgcBinnedSelectKnnRagged, or an empty tensor for the caller's order
        OP_REQUIRES(ctx, order.dim_size(0) == n_vert || order.dim_size(0) == 0,
                    errors::InvalidArgument("HgcGravnetCollect expects an order of length nvert or an empty one."));
        Tensor *out, *maxidx;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n_vert, 2 * F}, &out));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n_vert, F}, &maxidx));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_gravnet_collect(
            dist.flat<float>().data(), idx.flat<int>().data(), ld, first_slot_, ld - first_slot_,
            feat.flat<float>().data(), out->flat<float>().data(), 2 * F, maxidx->flat<int>().data(), n_vert, F,
            scale_, subtract_self_, order.dim_size(0) == n_vert ? order.flat<int>().data() : nullptr, StreamOf(ctx)),
            "HgcGravnetCollect"));
    }
private:
    int first_slot_;
    float scale_;
    bool subtract_self_;
};

// BuildAndAssignCondensatesBinned of modules/assign_condensate_op.py:210-310 (without keep_noise).
// alpha_idx comes back [N] with -1 after the last condensate; the wrapper slices it with
// n_condensates[-1], which TensorFlow reads on the host anyway.
class HgcBuildAndAssignCondensatesGpuOp : public OpKernel {
public:
    explicit HgcBuildAndAssignCondensatesGpuOp(OpKernelConstruction *c) : OpKernel(c) {
        OP_REQUIRES_OK(c, c->GetAttr("beta_threshold", &beta_threshold_));
        OP_REQUIRES_OK(c, c->GetAttr("distance_threshold", &distance_threshold_));
        OP_REQUIRES_OK(c, c->GetAttr("assign_by_max_beta", &assign_by_max_beta_));
        OP_REQUIRES_OK(c, c->GetAttr("nbin_dims", &nbin_dims_));
    }
    void Compute(OpKernelContext *ctx) override {
        const Tensor &cc = ctx->input(0), &betas = ctx->input(1), &dist = ctx->input(2), &mask = ctx->input(3),
                     &rs = ctx->input(4);
        const int n = cc.dim_size(0), dims = cc.dim_size(1), n_rs = rs.dim_size(0);
        Tensor *assignment, *asso, *alpha, *is_cond, *ncond;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, {n}, &assignment));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, {n}, &asso));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(2, {n}, &alpha));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(3, {n}, &is_cond));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(4, {n_rs}, &ncond));
        Workspace ws;
        OP_REQUIRES_OK(ctx, ws.Allocate(ctx, hgc_build_and_assign_condensates_workspace_bytes(n, dims, n_rs, nbin_dims_)));
        OP_REQUIRES_OK(ctx, FromHgc(hgc_build_and_assign_condensates(
            cc.flat<float>().data(), betas.flat<float>().data(), dist.flat<float>().data(),
            mask.dim_size(0) == n ? mask.flat<int>().data() : nullptr, rs.flat<int>().data(),
            assignment->flat<int>().data(), asso->flat<int>().data(), alpha->flat<int>().data(),
            is_cond->flat<uint8>().data(), ncond->flat<int>().data(), nullptr, n, dims, n_rs, beta_threshold_,
            distance_threshold_, assign_by_max_beta_, nbin_dims_, ws.ptr, ws.bytes, StreamOf(ctx)),
            "HgcBuildAndAssignCondensates"));
    }
private:
    float beta_threshold_, distance_threshold_;
    bool assign_by_max_beta_;
    int nbin_dims_;
};

}  // namespace

// Op signatures: identical to the reference's *_module.cc files.
REGISTER_OP("BinByCoordinates").Attr("calc_n_per_bin: bool")
    .Input("coordinates: float").Input("row_splits: int32").Input("bin_width: float").Input("nbins: int32")
    .Output("bin_assignment: int32").Output("flat_bin_assignment: int32").Output("nperbin: int32");
REGISTER_OP("BinnedSelectKnn").Attr("n_neighbours: int").Attr("tf_compatible: bool").Attr("use_direction: bool")
    .Input("coords: float").Input("bin_idx: int32").Input("dim_bin_idx: int32").Input("bin_boundaries: int32")
    .Input("n_bins: int32").Input("bin_width: float").Input("direction: int32")
    .Output("indices: int32").Output("distances: float32");
REGISTER_OP("IndexReplacer").Input("to_be_replaced: int32").Input("replacements: int32").Output("output: int32");
REGISTER_OP("AccumulateKnn").Attr("n_moments: int").Attr("mean_and_max: bool")
    .Input("distances: float32").Input("features: float32").Input("indices: int32")
    .Output("out_features: float32").Output("out_max_idxs: int32");
REGISTER_OP("AccumulateKnnGrad")
    .Input("grad_from_out_features: float32").Input("distances: float32").Input("features: float32")
    .Input("neigh_indices: int32").Input("max_feat_indices: int32")
    .Output("out_grad_distances: float32").Output("out_grad_features: float32");
REGISTER_OP("SelectKnnGrad")
    .Input("grad_distances: float32").Input("indices: int32").Input("distances: float32")
    .Input("coordinates: float32").Output("grad_coords: float32");
REGISTER_OP("LocalDistance").Input("coordinates: float32").Input("neighbour_idxs: int32").Output("distances: float32");
REGISTER_OP("PushKnn").Input("weights: float32").Input("features: float32").Input("indices: int32")
    .Output("out_features: float32");
REGISTER_OP("BinnedAssignToCondensates").Attr("beta_threshold: float").Attr("assign_by_max_beta: bool")
    .Input("ccoords: float32").Input("dist: float32").Input("beta: float32").Input("no_condensation_mask: int32")
    .Input("bins_flat: int32").Input("bin_splits: int32").Input("indices_to_filtered: int32")
    .Input("original_indices: int32").Input("row_splits: int32").Input("n_bins: int32").Input("bin_widths: float32")
    .Input("ccoords_h: float32").Input("dist_h: float32").Input("beta_h: float32")
    .Input("no_condensation_mask_h: int32").Input("row_splits_h: int32")
    .Output("assigned_h: int32").Output("assigned: int32").Output("alpha_indices: int32")
    .Output("association: int32").Output("n_condensates: int32");
// wrapper-level ops (no counterpart in the reference)
REGISTER_OP("HgcBinnedSelectKnnRagged").Attr("n_neighbours: int").Attr("n_bins: int = 0").Attr("max_bin_dims: int = 3")
    .Attr("tf_compatible: bool = false").Attr("use_direction: bool = false")
    .Input("coords: float").Input("row_splits: int32").Input("direction: int32")
    .Output("indices: int32").Output("distances: float32").Output("sorting: int32");
REGISTER_OP("HgcGravnetCollect").Attr("first_slot: int = 0").Attr("distance_scale: float = 10.0")
    .Attr("subtract_self: bool = true")
    .Input("distancesq: float32").Input("features: float32").Input("indices: int32")
    .Output("out_features: float32").Output("out_max_idxs: int32");
REGISTER_OP("HgcBuildAndAssignCondensates").Attr("beta_threshold: float").Attr("distance_threshold: float = 1.0")
    .Attr("assign_by_max_beta: bool = false").Attr("nbin_dims: int = 3")
    .Input("ccoords: float32").Input("betas: float32").Input("dist: float32").Input("no_condensation_mask: int32")
    .Input("row_splits: int32")
    .Output("assignment: int32").Output("association: int32").Output("alpha_idx: int32").Output("is_cond: uint8")
    .Output("n_condensates: int32");

REGISTER_KERNEL_BUILDER(Name("BinByCoordinates").Device(DEVICE_GPU).HostMemory("nbins").HostMemory("bin_width"),
                        BinByCoordinatesGpuOp);
REGISTER_KERNEL_BUILDER(Name("BinnedSelectKnn").Device(DEVICE_GPU), BinnedSelectKnnGpuOp);
REGISTER_KERNEL_BUILDER(Name("IndexReplacer").Device(DEVICE_GPU), IndexReplacerGpuOp);
REGISTER_KERNEL_BUILDER(Name("AccumulateKnn").Device(DEVICE_GPU), AccumulateKnnGpuOp);
REGISTER_KERNEL_BUILDER(Name("AccumulateKnnGrad").Device(DEVICE_GPU), AccumulateKnnGradGpuOp);
REGISTER_KERNEL_BUILDER(Name("SelectKnnGrad").Device(DEVICE_GPU), SelectKnnGradGpuOp);
REGISTER_KERNEL_BUILDER(Name("LocalDistance").Device(DEVICE_GPU), LocalDistanceGpuOp);
REGISTER_KERNEL_BUILDER(Name("PushKnn").Device(DEVICE_GPU), PushKnnGpuOp);
REGISTER_KERNEL_BUILDER(Name("BinnedAssignToCondensates").Device(DEVICE_GPU), BinnedAssignToCondensatesGpuOp);
REGISTER_KERNEL_BUILDER(Name("HgcBinnedSelectKnnRagged").Device(DEVICE_GPU), HgcBinnedSelectKnnRaggedGpuOp);
REGISTER_KERNEL_BUILDER(Name("HgcGravnetCollect").Device(DEVICE_GPU), HgcGravnetCollectGpuOp);
REGISTER_KERNEL_BUILDER(Name("HgcBuildAndAssignCondensates").Device(DEVICE_GPU), HgcBuildAndAssignCondensatesGpuOp);

}  // namespace tensorflow
