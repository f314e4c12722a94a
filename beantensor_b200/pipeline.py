"""Two sharded products in a row, pipelined by row panels: GEMM -> all-gather -> next GEMM.

Layer 1 is the N-sharded product with the all-gather fused into its epilogue (every rank ends up with all of
C1 = A . B1); layer 2 multiplies C1 by this rank's column block of B2. Run as two whole products, layer 2 cannot start
before the last tile of layer 1 has landed on every rank and a cross-rank barrier has passed, so the tail of layer 1's
all-gather and the barrier are exposed once per layer. Run by row panels they are hidden: as soon as the rows of panel p
are complete everywhere, layer 2 multiplies those rows while layer 1 is already working on panel p + 1.

Three streams, no kernel ever waits on another kernel's progress by itself (only stream order and events):
  s1  layer-1 products, panel after panel;
  s3  after each panel of s1, a one-element all-reduce (the cross-rank "panel p has landed everywhere");
  s2  layer-2 products, panel p after s3's event p.
The reference has no operator graph to fuse (its Ops are free functions that run one after the other); this is the
scheduling a BeanTensor caller with two matmul layers would write by hand on top of the operators.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .errors import raise_for_status


class TwoLayerNShard:
    """C2[:, block] = (A . B1) . B2[:, block] over `world` ranks; C1 is gathered on every rank on the way.

    a          [M, K1] on this rank (replicated operand)
    b1_block   [K1, N1/world] this rank's column block of B1
    b2_block   [N1, N2/world] this rank's column block of B2
    c1_local / c1_peer: where layer 1 stores. Either (local pointer, multicast pointer) of a MulticastBuffer, or
               (table of every rank's C1 base, None) for plain peer stores.
    c2         [M, N2/world] output block of this rank
    """

    def __init__(self, dist, device, rank, world, dtype_code, a, b1_block, b2_block, c1_local_ptr, c1_mc_ptr, c1_table, c1_view, c2, panels):
        self.L = _lib.lib()
        self.dist, self.dev, self.rank, self.world, self.dt = dist, device, rank, world, dtype_code
        self.a, self.b1, self.b2, self.c1, self.c2 = a, b1_block, b2_block, c1_view, c2
        self.c1_local_ptr, self.c1_mc_ptr, self.c1_table = c1_local_ptr, c1_mc_ptr, c1_table
        self.M, self.K1 = a.shape
        self.n1loc = b1_block.shape[1]
        self.N1 = self.n1loc * world
        self.n2loc = b2_block.shape[1]
        if self.M % panels:
            raise ValueError("rows must divide into the panels")
        self.panels, self.mp = panels, self.M // panels
        self.s1, self.s2, self.s3 = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        self.flag = torch.zeros(1, dtype=torch.int32, device=a.device)
        self.es = a.element_size()

    def _layer1(self, stream, row0, rows):
        off = row0 * self.N1 * self.es
        a_ptr = self.a.data_ptr() + row0 * self.K1 * self.es
        st = C.c_void_p(stream.cuda_stream)
        if self.c1_mc_ptr is not None:
            rc = self.L.btm_gemm_nshard_mc(self.dev, st, self.dt, rows, self.n1loc, self.K1, a_ptr, self.K1, self.b1.data_ptr(), self.n1loc,
                                           self.c1_local_ptr + off, self.c1_mc_ptr + off, self.N1, self.rank, self.world)
        else:
            table = (C.c_void_p * self.world)(*[p + off for p in self.c1_table])
            rc = self.L.btm_gemm_nshard(self.dev, st, self.dt, rows, self.n1loc, self.K1, a_ptr, self.K1, self.b1.data_ptr(), self.n1loc,
                                        table, self.N1, self.rank, self.world)
        raise_for_status(rc)

    def _layer2(self, stream, row0, rows):
        st = C.c_void_p(stream.cuda_stream)
        rc = self.L.btm_gemm(self.dev, st, self.dt, rows, self.n2loc, self.N1, self.c1.data_ptr() + row0 * self.N1 * self.es, self.N1,
                             self.b2.data_ptr(), self.n2loc, self.c2.data_ptr() + row0 * self.n2loc * self.es, self.n2loc)
        raise_for_status(rc)

    def run_sequential(self):
        """Two whole products with a barrier between them, on the current stream."""
        cur = torch.cuda.current_stream()
        self._layer1(cur, 0, self.M)
        self.dist.all_reduce(self.flag)   # stream-ordered: every rank's tiles of C1 have landed
        self._layer2(cur, 0, self.M)
        self.dist.all_reduce(self.flag)   # nobody overwrites C1 (next step) while a rank still reads it

    def run_pipelined(self):
        cur = torch.cuda.current_stream()
        for s in (self.s1, self.s2, self.s3):
            s.wait_stream(cur)
        for p in range(self.panels):
            row0 = p * self.mp
            self._layer1(self.s1, row0, self.mp)
            done = torch.cuda.Event()
            done.record(self.s1)
            self.s3.wait_event(done)
            with torch.cuda.stream(self.s3):
                self.dist.all_reduce(self.flag)          # panel p of C1 is complete on every rank
                landed = torch.cuda.Event()
                landed.record(self.s3)
            self.s2.wait_event(landed)
            self._layer2(self.s2, row0, self.mp)
        cur.wait_stream(self.s1)
        cur.wait_stream(self.s2)
        cur.wait_stream(self.s3)
        self.dist.all_reduce(self.flag)   # as in run_sequential: C1 may be rewritten after this
