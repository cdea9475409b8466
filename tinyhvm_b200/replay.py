"""Replay of a recorded training step against the vtable C ABI.

A trace is the exact sequence of `Backend` calls the reference's host runtime
(reducer, fuser, scheduler) makes for a staged training program: buf_alloc,
buf_write, dispatch_kernel_rs with every view / op / reduce spec, buf_copy,
decref/free, pool_reset.  Replaying it drives libthvm_cuda.so with exactly what
the reference's scheduler would send, step after step, without the host
interaction-net reduction: the analogue of the capture/replay JIT of the
reference's Metal backend (src/backend/metal/jit.m:24-631,
src/tinyhvm.h:1294-1300), and the way the CNN training configs are benchmarked
here.  Traces are recorded by oracle/ref_trace.c (test infrastructure, needs the
reference checkout) and committed under tinyhvm_b200/traces/.

`Replayer.capture` records a cycle once as a CUDA graph (CapturedStep); every later
step is then a single graph launch.

Layout of a trace: 8-byte header, then records `u32 op, u32 bytes, payload`.
Host writes larger than 8 KiB, and the ones the driver named (inputs, one-hot
labels, parameters, the learning rate), carry no data: the caller supplies them
per step through `externals[name]`.
"""
from __future__ import annotations

import ctypes as C
import gzip
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import numpy as np

from . import abi

(ALLOC, WRITE, READ, DISPATCH, COPY, CONTIGUIFY, FREE, INCREF, DECREF, POOL_RESET, SET_PERSISTENT, ALLREDUCE, MARK) = range(1, 14)
SGD_FUSED = 100                      # not a trace record: made by fuse_optimizer from an all-reduce and its update dispatches
TRACE_DIR = Path(__file__).resolve().parent / "traces"


@dataclass
class Record:
    op: int
    f: tuple                      # decoded fields
    blob: bytes = b""             # inline write payload / raw dispatch payload


def load_trace(path) -> list[Record]:
    path = Path(path)
    data = gzip.open(path, "rb").read() if path.suffix == ".gz" else path.read_bytes()
    magic, version = struct.unpack_from("<II", data, 0)
    assert magic == 0x52544854 and version == 1, "not a vtable trace"
    pos, out = 8, []
    while pos < len(data):
        op, n = struct.unpack_from("<II", data, pos)
        pos += 8
        p = data[pos:pos + n]
        pos += n
        if op == ALLOC or op == READ:
            i, _, nb = struct.unpack_from("<IIQ", p, 0)
            out.append(Record(op, (i, nb)))
        elif op == WRITE:
            i, ext, nb = struct.unpack_from("<IIQ", p, 0)
            name = p[16:48].split(b"\0")[0].decode()
            out.append(Record(op, (i, ext, nb, name), p[48:48 + nb] if not ext else b""))
        elif op == DISPATCH:
            out.append(Record(op, (), p))
        elif op == COPY:
            out.append(Record(op, struct.unpack_from("<IIQ", p, 0)))
        elif op in (FREE, INCREF, DECREF, POOL_RESET, SET_PERSISTENT):
            out.append(Record(op, struct.unpack_from("<I", p, 0)))
        elif op == ALLREDUCE:
            (k,) = struct.unpack_from("<I", p, 0)
            ids = struct.unpack_from(f"<{k}I", p, 4)
            counts = struct.unpack_from(f"<{k}Q", p, 4 + 4 * k)
            out.append(Record(op, (ids, counts)))
        elif op == MARK:
            out.append(Record(op, (p[:32].split(b"\0")[0].decode(),)))
        else:
            raise ValueError(f"unknown trace op {op}")
    return out


def split_steps(recs: list[Record]):
    """(prefix, [cycle0, cycle1, ...]): a cycle runs from one step_begin mark to the next."""
    starts = [i for i, r in enumerate(recs) if r.op == MARK and r.f[0] == "step_begin"]
    assert starts, "trace holds no step"
    cycles = [recs[a:b] for a, b in zip(starts, starts[1:] + [len(recs)])]
    return recs[:starts[0]], cycles


class DispatchArgs:
    """ctypes arguments of one recorded dispatch_kernel_rs call, built once."""

    def __init__(self, blob: bytes):
        out, n, n_ops, out_dt, has_red, has_sts = struct.unpack_from("<6I", blob, 0)
        pos = 24
        self.full = abi.Shape.from_buffer_copy(blob, pos); pos += C.sizeof(abi.Shape)
        self.red = abi.ReduceSpec.from_buffer_copy(blob, pos); pos += C.sizeof(abi.ReduceSpec)
        self.ids = (C.c_uint32 * n).from_buffer_copy(blob, pos); pos += 4 * n
        self.dts = (C.c_uint32 * n).from_buffer_copy(blob, pos); pos += 4 * n
        self.views = (abi.View * n).from_buffer_copy(blob, pos); pos += C.sizeof(abi.View) * n
        self.ops = (abi.FusedOp * max(n_ops, 1)).from_buffer_copy(blob[pos:pos + 16 * n_ops].ljust(16, b"\0")); pos += 16 * n_ops
        self.view_ptrs = (C.POINTER(abi.View) * n)(*[C.pointer(self.views[i]) for i in range(n)])
        self.sts, self.st_ptrs = None, None
        if has_sts:
            self.sts, ptrs = [], (C.POINTER(abi.Tracker) * n)()
            for i in range(n):
                present = blob[pos]; pos += 1
                if present:
                    t = abi.Tracker.from_buffer_copy(blob, pos); pos += C.sizeof(abi.Tracker)
                    self.sts.append(t)
                    ptrs[i] = C.pointer(t)
            self.st_ptrs = C.cast(ptrs, C.c_void_p)
            self._keep = ptrs
        self.out, self.n, self.n_ops, self.out_dt, self.has_red = out, n, n_ops, out_dt, has_red


class CudaTarget:
    """The product: libthvm_cuda.so through its C ABI."""

    def __init__(self, backend):
        self.be, self.lib = backend, backend.lib

    def alloc(self, nbytes): return self.lib.thvm_cuda_buf_alloc(nbytes)
    def write(self, i, ptr, nbytes): self.lib.thvm_cuda_buf_write(i, ptr, nbytes)
    def read(self, i, ptr, nbytes): self.lib.thvm_cuda_buf_read(i, ptr, nbytes)
    def copy(self, d, s, nbytes): self.lib.thvm_cuda_buf_copy(d, s, nbytes)
    def free(self, i): self.lib.thvm_cuda_buf_free(i)
    def incref(self, i): self.lib.thvm_cuda_buf_incref(i)
    def decref(self, i): self.lib.thvm_cuda_buf_decref(i)
    def pool_reset(self, keep): self.lib.thvm_cuda_pool_reset(keep)
    def set_persistent(self, m): self.lib.thvm_cuda_pool_set_persistent(m)

    def dispatch(self, a: DispatchArgs):
        self.lib.thvm_cuda_dispatch_kernel_rs(a.out, a.ids, a.view_ptrs, a.st_ptrs, a.n, a.ops, a.n_ops, C.byref(a.full),
                                              C.byref(a.red) if a.has_red else None, None, None, 0, a.dts, a.out_dt)

    def allreduce(self, ids, counts):
        k = len(ids)
        rc = self.lib.thvm_cuda_dp_allreduce_sum((C.c_uint32 * k)(*ids), (C.c_uint64 * k)(*counts), k)
        assert rc == 0, self.be.last_error()

    def sgd_step(self, params, grads, counts, lr_buf):
        k = len(params)
        rc = self.lib.thvm_cuda_dp_sgd_step((C.c_uint32 * k)(*params), (C.c_uint32 * k)(*grads), (C.c_uint64 * k)(*counts), k, lr_buf)
        assert rc == 0, self.be.last_error()


class CapturedStep:
    """One steady-state cycle of a trace recorded as a CUDA graph (thvm_cuda_capture_*): `launch(externals)`
    points the graph's inputs at this step's host arrays (keep them alive, ideally pinned, until the results
    have been fetched) and enqueues the whole step with one call; `results()` waits and returns the named
    reads.  The cycle must have been replayed eagerly before (plans built, scratch grown)."""

    def __init__(self, rp: "Replayer", recs, externals: dict):
        t = rp.t
        assert isinstance(t, CudaTarget), "step capture needs the CUDA library"
        self.lib, self.be = t.lib, t.be
        self.inputs, self.reads, used = [], [], {}
        assert self.lib.thvm_cuda_capture_begin() == 0, self.be.last_error()
        for item in rp._bind(recs):
            kind = item[0]
            if kind == "call":
                item[1](*item[2])
            elif kind == "alloc":
                got = t.alloc(item[2])
                assert got == item[1], f"buffer id {got} where the trace has {item[1]}: pool out of step with the recording"
            elif kind == "ext":
                _, i, nb, name = item
                k = used.get(name, 0); used[name] = k + 1
                src = externals[name]
                src = src[k % len(src)] if isinstance(src, (list, tuple)) else src
                assert src.nbytes == nb, f"external {name}: {src.nbytes} bytes supplied, trace wants {nb}"
                idx = self.lib.thvm_cuda_capture_input(i, src.ctypes.data, nb)
                assert idx == len(self.inputs), self.be.last_error()
                self.inputs.append((name, k, nb))
            elif kind == "read":
                _, i, nb, name = item
                scratch = np.empty(nb, dtype=np.uint8)
                t.read(i, scratch.ctypes.data, nb)          # recorded as a result of the graph (or served from a host shadow)
                self.reads.append((name, nb))
        self.handle = self.lib.thvm_cuda_capture_end()
        assert self.handle > 0, self.be.last_error()
        ni, nr, nk = C.c_uint32(), C.c_uint32(), C.c_uint64()
        self.lib.thvm_cuda_graph_counts(self.handle, C.byref(ni), C.byref(nr), C.byref(nk))
        assert ni.value == len(self.inputs)
        self.n_results, self.n_kernels = nr.value, nk.value
        # reads that were served from a host shadow never became graph results; the trace's training steps have none
        assert self.n_results == len(self.reads), "a read inside the captured step did not come from the device"

    def launch(self, externals: dict):
        self._alive = []
        for idx, (name, k, nb) in enumerate(self.inputs):
            src = externals[name]
            src = src[k % len(src)] if isinstance(src, (list, tuple)) else src
            assert src.nbytes == nb
            self._alive.append(src)
            assert self.lib.thvm_cuda_graph_set_input(self.handle, idx, src.ctypes.data) == 0, self.be.last_error()
        assert self.lib.thvm_cuda_graph_launch(self.handle) == 0, self.be.last_error()

    def prefetch(self, externals: dict) -> None:
        """Upload the NEXT launch's inputs now, on the library's copy stream, while the step just launched runs; follow
        with `launch_prefetched()`.  The arrays must stay alive and unchanged until that launch has started."""
        self._next = []
        for idx, (name, k, nb) in enumerate(self.inputs):
            src = externals[name]
            src = src[k % len(src)] if isinstance(src, (list, tuple)) else src
            assert src.nbytes == nb
            self._next.append(src)
            assert self.lib.thvm_cuda_graph_prefetch_input(self.handle, idx, src.ctypes.data) == 0, self.be.last_error()

    def launch_prefetched(self) -> None:
        self._alive = self._next
        assert self.lib.thvm_cuda_graph_launch(self.handle) == 0, self.be.last_error()

    def results_async(self, outs: dict) -> None:
        """Queue copies of the named results of the latest launch into the caller's pinned arrays (`outs[name]`);
        they are valid once the stream has passed this point."""
        for k, (name, nb) in enumerate(self.reads):
            if name in outs:
                assert self.lib.thvm_cuda_graph_result_async(self.handle, k, outs[name].ctypes.data, min(nb, outs[name].nbytes)) == 0, self.be.last_error()

    def results(self) -> dict:
        out = {}
        for k, (name, nb) in enumerate(self.reads):
            buf = np.empty(nb, dtype=np.uint8)
            assert self.lib.thvm_cuda_graph_result(self.handle, k, buf.ctypes.data, nb) == 0, self.be.last_error()
            if name:
                out[name] = buf.view(np.float32) if nb % 4 == 0 else buf
        return out

    def destroy(self):
        if self.handle:
            self.lib.thvm_cuda_graph_destroy(self.handle)
            self.handle = 0


def fuse_optimizer(recs: list[Record]) -> list[Record]:
    """Rewrite the optimizer tail of a recorded step for `thvm_cuda_dp_sgd_step`.

    The staged step ends with the gradient all-reduce followed, per parameter tensor, by the dispatch
    T = p - g * lr and the ASSIGN copy p <- T (src/interact/tensor_ops.c:93-147).  Where exactly that shape is found —
    every all-reduced gradient feeds one such dispatch, whose result is copied over its first leaf — the all-reduce,
    the dispatches and the copies are replaced by ONE fused record (parameter ids, gradient ids, counts, the buffer
    holding lr), placed where the last copy stood.  Allocations, constant writes and frees stay as recorded, so buffer
    ids keep matching.  Anything else is returned unchanged."""
    ar = [k for k, r in enumerate(recs) if r.op == ALLREDUCE]
    if len(ar) != 1:
        return recs
    grads, counts = recs[ar[0]].f
    want = {g: n for g, n in zip(grads, counts)}
    found, drop, last = {}, {ar[0]}, None
    k = ar[0] + 1
    while k < len(recs):
        r = recs[k]
        if r.op == DISPATCH:
            a = DispatchArgs(r.blob)
            ops = [(a.ops[i].uop, a.ops[i].arg_a, a.ops[i].arg_b) for i in range(a.n_ops)]
            if a.n == 3 and ops == [(abi.MUL, 1, 2), (abi.SUB, 0, 3)] and not a.has_red and a.ids[1] in want and a.ids[1] not in found:
                numel = 1
                for d in range(a.full.rank):
                    numel *= a.full.dims[d]
                flat = all(a.views[i].contiguous and a.views[i].offset == 0 for i in range(2)) and a.views[2].offset == 0 and \
                    all(a.views[2].strides[d] == 0 or a.views[2].shape.dims[d] == 1 for d in range(a.views[2].shape.rank))
                nxt = next((j for j in range(k + 1, len(recs)) if recs[j].op in (COPY, DISPATCH, ALLREDUCE)), None)
                if flat and numel == want[a.ids[1]] and nxt is not None and recs[nxt].op == COPY and recs[nxt].f[0] == a.ids[0] \
                        and recs[nxt].f[1] == a.out and recs[nxt].f[2] == 4 * numel:
                    found[a.ids[1]] = (a.ids[0], a.ids[2])
                    drop |= {k, nxt}
                    last = nxt
        k += 1
    if set(found) != set(want) or last is None or len({lr for _, lr in found.values()}) < 1:
        return recs
    params = tuple(found[g][0] for g in grads)
    lr_buf = found[grads[-1]][1]          # every tensor's step size is the same external; the last one written is live at the fused call
    out = []
    for k, r in enumerate(recs):
        if k == last:
            out.append(Record(SGD_FUSED, (params, tuple(grads), tuple(counts), lr_buf)))
        elif k not in drop:
            out.append(r)
    return out


class Replayer:
    """Binds a trace to a target once; `run(cycle, externals)` then replays one cycle.

    `externals[name]` is a numpy array, or a list of arrays consumed in order when
    the cycle writes that name several times.  `fused_optimizer=True` replays the optimizer tail of every step
    through one fused all-reduce + SGD call (see fuse_optimizer)."""

    def __init__(self, target, recs: list[Record], fused_optimizer: bool = False):
        self.t = target
        self.prefix, self.cycles = split_steps(recs)
        if fused_optimizer:
            self.cycles = [fuse_optimizer(c) for c in self.cycles]
        self._bound = {}

    def _bind(self, recs):
        key = id(recs)
        if key in self._bound:
            return self._bound[key]
        t, prog, pending = self.t, [], None
        for r in recs:
            if r.op == ALLOC:
                prog.append(("alloc", r.f[0], r.f[1]))
            elif r.op == WRITE:
                i, ext, nb, name = r.f
                if ext:
                    prog.append(("ext", i, nb, name))
                else:
                    buf = C.create_string_buffer(r.blob, max(len(r.blob), 1))
                    prog.append(("call", t.write, (i, C.cast(buf, C.c_void_p), nb), buf))
            elif r.op == READ:
                prog.append(("read", r.f[0], r.f[1], pending)); pending = None
            elif r.op == DISPATCH:
                prog.append(("call", t.dispatch, (DispatchArgs(r.blob),), None))
            elif r.op == COPY:
                prog.append(("call", t.copy, tuple(r.f), None))
            elif r.op == FREE:
                prog.append(("call", t.free, tuple(r.f), None))
            elif r.op == INCREF:
                prog.append(("call", t.incref, tuple(r.f), None))
            elif r.op == DECREF:
                prog.append(("call", t.decref, tuple(r.f), None))
            elif r.op == POOL_RESET:
                prog.append(("call", t.pool_reset, tuple(r.f), None))
            elif r.op == SET_PERSISTENT:
                prog.append(("call", t.set_persistent, tuple(r.f), None))
            elif r.op == ALLREDUCE:
                prog.append(("call", t.allreduce, tuple(r.f), None))
            elif r.op == SGD_FUSED:
                prog.append(("call", t.sgd_step, tuple(r.f), None))
            elif r.op == MARK and r.f[0].startswith("read:"):
                pending = r.f[0][5:]
        self._bound[key] = prog
        return prog

    def run(self, recs, externals: dict) -> dict:
        t, reads, used = self.t, {}, {}
        for item in self._bind(recs):
            kind = item[0]
            if kind == "call":
                item[1](*item[2])
            elif kind == "alloc":
                got = t.alloc(item[2])
                assert got == item[1], f"buffer id {got} where the trace has {item[1]}: pool out of step with the recording"
            elif kind == "ext":
                _, i, nb, name = item
                src = externals[name]
                if isinstance(src, (list, tuple)):
                    k = used.get(name, 0); used[name] = k + 1
                    src = src[k % len(src)]
                assert src.nbytes == nb, f"external {name}: {src.nbytes} bytes supplied, trace wants {nb}"
                t.write(i, src.ctypes.data, nb)
            elif kind == "read":
                _, i, nb, name = item
                out = np.empty(nb, dtype=np.uint8)
                t.read(i, out.ctypes.data, nb)
                if name:
                    reads[name] = out.view(np.float32) if nb % 4 == 0 else out
        return reads

    def capture(self, recs, externals: dict) -> CapturedStep:
        return CapturedStep(self, recs, externals)

    def run_prefix(self, externals: dict) -> dict:
        return self.run(self.prefix, externals)

    def n_dispatches(self, recs) -> int:
        return sum(1 for r in recs if r.op == DISPATCH)
