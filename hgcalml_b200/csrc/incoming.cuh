// Transposed neighbour lists: for every hit, the (hit, slot) edges that point at it, in ascending
// (hit, slot) order.  Built with the stable counting sort, used by the ops that push values from a
// hit to its neighbours (backward ops, PushKnn) so that they need no atomics.
#pragma once
#include "common.cuh"

namespace hgc {

struct Incoming {
    int *keys, *skeys, *sedges, *tkeys, *tvals, *hist, *bounds;
};

template <typename W>
Incoming incoming_layout(W &ws, int n_vert, int n_neigh)
{
    const size_t ne = (size_t)(n_vert > 0 ? n_vert : 0) * (size_t)(n_neigh > 0 ? n_neigh : 0);
    Incoming b;
    b.keys = ws.template take<int>(ne);
    b.skeys = ws.template take<int>(ne);
    b.sedges = ws.template take<int>(ne);
    b.tkeys = ws.template take<int>(ne);
    b.tvals = ws.template take<int>(ne);
    b.hist = ws.template take<int>(sort_hist_ints((int)ne));
    b.bounds = ws.template take<int>((size_t)(n_vert > 0 ? n_vert : 0) + 2);
    return b;
}

struct IncomingSizer {
    Sizer s;
    template <typename T> T *take(size_t n) { s.take<T>(n); return nullptr; }
};

// bounds[m] .. bounds[m+1]: positions in sedges of the edges whose neighbour is hit m; sedges holds
// edge ids e = hit * n_neigh + slot.
int build_incoming(const int *nidx, int n_vert, int n_neigh, const Incoming &b, cudaStream_t stream);

}  // namespace hgc
