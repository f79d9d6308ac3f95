"""BinnedSelectKnn + AccumulateKnn for batches that live in HOST memory.

Events are independent, so a ragged batch is cut into chunks of whole events and the chunks flow
through three stages on three CUDA streams -- host->device copy of coordinates, features and row
splits; the two ops; device->host copy of the accumulated features -- with double-buffered device
inputs, so the PCIe transfers of neighbouring chunks overlap the kernels of the current one.
Results are those of one call over the whole batch: the binning grid is derived per chunk, and the
neighbour search does not depend on the grid.
"""
from __future__ import annotations

import numpy as np
import torch

from .accknn_op import AccumulateKnn
from .binned_select_knn_op import BinnedSelectKnn


class KnnAccumulatePipeline:
    def __init__(self, K: int, device, events_per_chunk: int = 2, distance_scale: float = 10.,
                 n_slots: int = 2, with_max_idxs: bool = False):
        self.K = int(K)
        self.device = torch.device(device)
        self.events_per_chunk = max(1, int(events_per_chunk))
        self.distance_scale = float(distance_scale)
        self.n_slots = max(2, int(n_slots))
        self.with_max_idxs = with_max_idxs
        self.s_h2d = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_d2h = torch.cuda.Stream(self.device)
        self._slots = None
        self._rs_pinned = None
        self._h2d_done = None

    def _ensure_slots(self, max_hits, n_coords, n_feat, max_events):
        ok = (self._slots is not None and self._slots[0]["coords"].shape[0] >= max_hits
              and self._slots[0]["coords"].shape[1] == n_coords and self._slots[0]["feats"].shape[1] == n_feat
              and self._slots[0]["rs"].shape[0] >= max_events + 1)
        if ok:
            return
        self._slots = []
        for _ in range(self.n_slots):
            self._slots.append(dict(
                coords=torch.empty((max_hits, n_coords), dtype=torch.float32, device=self.device),
                feats=torch.empty((max_hits, n_feat), dtype=torch.float32, device=self.device),
                rs=torch.empty((max_events + 1,), dtype=torch.int32, device=self.device),
                coords_loaded=torch.cuda.Event(), loaded=torch.cuda.Event(), consumed=torch.cuda.Event()))
            self._slots[-1]["consumed"].record(torch.cuda.current_stream(self.device))

    def run(self, coords: torch.Tensor, feats: torch.Tensor, row_splits, out: torch.Tensor, wait: bool = True,
            copies_only: bool = False):
        """coords [N,C], feats [N,F]: pinned host float32 tensors; row_splits: host int array [E+1];
        out [N,2F]: pinned host float32 tensor that receives [mean | max].

        With ``wait`` (the default) the call returns once every row of ``out`` has arrived in host
        memory (the device-to-host stream is synchronised).  With ``wait=False`` it returns as soon
        as the work is enqueued: the caller's current CUDA stream then waits for the three pipeline
        streams, but the host does not, so ``out`` must not be read before that stream (or the
        device) has been synchronised.

        ``copies_only`` skips the two ops and moves the same bytes through the same buffers, streams
        and events (the result rows are whatever the staging buffer holds): the transfer-only time of
        the pipeline, against which the full call can be compared."""
        rs = np.asarray(row_splits, dtype=np.int64)
        n_events = len(rs) - 1
        chunks = [(e0, min(e0 + self.events_per_chunk, n_events))
                  for e0 in range(0, n_events, self.events_per_chunk)]
        max_hits = max(int(rs[e1] - rs[e0]) for e0, e1 in chunks) if chunks else 0
        self._ensure_slots(max_hits, coords.shape[1], feats.shape[1], self.events_per_chunk)
        start = torch.cuda.current_stream(self.device)
        for s in (self.s_h2d, self.s_run, self.s_d2h):
            s.wait_stream(start)
        # row splits of all chunks, rebased to their chunk, in one pinned buffer that is kept between calls
        width = self.events_per_chunk + 1
        if self._rs_pinned is None or self._rs_pinned.shape[0] < len(chunks):
            self._rs_pinned = torch.empty((max(len(chunks), 1), width), dtype=torch.int32).pin_memory()
        if self._h2d_done is not None:
            self._h2d_done.synchronize()  # the previous call's copies out of this buffer have finished
        rs_host = self._rs_pinned.numpy()
        for c, (e0, e1) in enumerate(chunks):
            rs_host[c, :e1 - e0 + 1] = rs[e0:e1 + 1] - rs[e0]
        rs_chunks = [self._rs_pinned[c, :e1 - e0 + 1] for c, (e0, e1) in enumerate(chunks)]
        for c, (e0, e1) in enumerate(chunks):
            slot = self._slots[c % self.n_slots]
            lo, hi = int(rs[e0]), int(rs[e1])
            n = hi - lo
            with torch.cuda.stream(self.s_h2d):
                self.s_h2d.wait_event(slot["consumed"])
                # coordinates and row splits first: the search can start while the (16 times larger)
                # features of the same chunk are still on their way
                slot["coords"][:n].copy_(coords[lo:hi], non_blocking=True)
                slot["rs"][:e1 - e0 + 1].copy_(rs_chunks[c], non_blocking=True)
                slot["coords_loaded"].record(self.s_h2d)
                slot["feats"][:n].copy_(feats[lo:hi], non_blocking=True)
                slot["loaded"].record(self.s_h2d)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(slot["coords_loaded"])
                if copies_only:
                    self.s_run.wait_event(slot["loaded"])
                    res = torch.empty((n, 2 * feats.shape[1]), dtype=torch.float32, device=self.device)
                else:
                    idx, d2, sorting = BinnedSelectKnn(self.K, slot["coords"][:n], slot["rs"][:e1 - e0 + 1],
                                                       return_sorting=True)
                    self.s_run.wait_event(slot["loaded"])
                    res, _ = AccumulateKnn(d2, slot["feats"][:n], idx, order=sorting,
                                           distance_scale=self.distance_scale, with_max_idxs=self.with_max_idxs)
                slot["consumed"].record(self.s_run)
                done = torch.cuda.Event()
                done.record(self.s_run)
            with torch.cuda.stream(self.s_d2h):
                self.s_d2h.wait_event(done)
                out[lo:hi].copy_(res, non_blocking=True)
                res.record_stream(self.s_d2h)
        self._h2d_done = torch.cuda.Event()
        self._h2d_done.record(self.s_h2d)
        start.wait_stream(self.s_d2h)
        start.wait_stream(self.s_run)
        start.wait_stream(self.s_h2d)
        if wait:
            self.s_d2h.synchronize()
        return out
