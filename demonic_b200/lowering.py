"""Kernel selection for one `@` site: the host logic the JIT runs at compile time.

A Python restatement, for this backend's flag, of what the reference's
``lower_matmul_general`` (compiler/src/jit.rs:19860-20032),
``emit_2d_matmul_bf16_at`` (compiler/src/jit.rs:20916-20946) and
``emit_2d_matmul_at`` (compiler/src/jit.rs:20806-20831) decide from static
shapes: broadcast the batch dims, test whether the per-slice offsets are affine
in the flat batch index, and pick the runtime symbol.  The flag follows the
``--blas`` rule (compiler/src/jit.rs:29346-29351): off by default and never
selected inside ``@deterministic``.

``lower`` is pure (no device).  ``run`` executes a plan's GPU calls through the
C ABI with raw host addresses, the way JIT-emitted code does; calls that stay
on the reference's own CPU builtins are returned to the caller untouched --
this package computes nothing on the CPU.
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field

import numpy as np

from . import _lib

GPU_MIN_MACS = 4_000_000          # compiler/src/jit.rs:20933
GPU_BATCH_MIN_MACS = 1_000_000    # compiler/src/jit.rs:19912
GPU_BATCH_MAX = 65_536            # compiler/src/jit.rs:19915
F32_MIN_MACS = 1 << 17            # BLAS_MIN_MACS, compiler/src/jit.rs:29340

SYM_BATCHED = "dmc_matmul_bf16_gpu_batched"
SYM_BATCHED_DEFERRED = "dmc_matmul_bf16_gpu_batched_deferred"
SYM_SINGLE = "dmc_matmul_bf16_gpu"
SYM_F32 = "dmc_matmul_f32_gpu"
SYM_FLUSH = "dmc_matmul_bf16_gpu_flush"
CPU_BF16 = "dmc_matmul_bf16"      # the reference's CPU builtins: not ours to run
CPU_F32 = "cpu_f32_matmul"


@dataclass
class Call:
    symbol: str
    l_off: int      # element offsets into the flat operands
    r_off: int
    out_off: int
    m: int
    k: int
    n: int
    batch: int = 1
    ls: int = 0
    rs: int = 0

    @property
    def on_gpu(self) -> bool:
        return self.symbol in (SYM_BATCHED, SYM_BATCHED_DEFERRED, SYM_SINGLE, SYM_F32)


@dataclass
class Plan:
    out_shape: tuple
    calls: list = field(default_factory=list)
    flush_first: bool = False


def _strides(shape):
    s, acc = [], 1
    for d in reversed(shape):
        s.append(acc)
        acc *= d
    return list(reversed(s))


class Lowering:
    """Per-function lowering state: the flag, the ``@deterministic`` nesting depth
    (compiler/src/jit.rs:8077-8083) and the deferred-call bookkeeping
    (compiler/src/jit.rs:8726-8744, 20903-20914)."""

    def __init__(self, cuda: bool = False):
        self.cuda = cuda                  # default off, like Jit.blas (compiler/src/jit.rs:39105-39113)
        self.deterministic_depth = 0
        self.defer_hint = False           # next statement is a batched candidate too
        self.defer_pending = False

    @contextmanager
    def deterministic(self):
        """``with_deterministic`` (compiler/src/jit.rs:20861-20868): a depth, not a flag."""
        self.deterministic_depth += 1
        try:
            yield self
        finally:
            self.deterministic_depth -= 1

    def _gpu_on(self) -> bool:
        return self.cuda and self.deterministic_depth == 0

    def lower(self, l_shape, r_shape, rhs_bf16: bool = True) -> Plan:
        l_shape, r_shape = tuple(l_shape), tuple(r_shape)
        if len(l_shape) < 2 or len(r_shape) < 2:
            raise ValueError("matmul `@` needs rank >= 2 on both sides")
        m, k = l_shape[-2:]
        k2, n = r_shape[-2:]
        if k != k2:
            raise ValueError(f"matmul inner dim mismatch: lhs [.., {k}] vs rhs [{k2}, ..]")
        lb, rb = l_shape[:-2], r_shape[:-2]
        rank = max(len(lb), len(rb))
        ob = []
        for i in range(rank):
            ld = lb[i - (rank - len(lb))] if i >= rank - len(lb) else 1
            rd = rb[i - (rank - len(rb))] if i >= rank - len(rb) else 1
            if ld != rd and ld != 1 and rd != 1:
                raise ValueError(f"matmul batch dims not broadcastable: {ld} vs {rd}")
            ob.append(max(ld, rd))
        total = int(np.prod(ob)) if ob else 1
        lmat, rmat, omat = m * k, k * n, m * n
        ob_s, lb_s, rb_s = _strides(ob), _strides(lb), _strides(rb)

        def flat(p, b, b_s):
            f = 0
            for ax in range(rank):
                coord = (p // ob_s[ax]) % ob[ax]
                if ax + len(b) >= rank:
                    a = ax + len(b) - rank
                    if b[a] > 1:
                        f += coord * b_s[a]
            return f

        plan = Plan(out_shape=tuple(ob) + (m, n))
        if self._gpu_on() and rhs_bf16 and m == 1 and n % 4 == 0 and total <= GPU_BATCH_MAX \
                and total * m * k * n >= GPU_BATCH_MIN_MACS:
            ls = flat(1, lb, lb_s) * lmat if total > 1 else 0
            rs = flat(1, rb, rb_s) * rmat if total > 1 else 0
            affine = rs % 4 == 0 and all(
                flat(p, lb, lb_s) * lmat == p * ls and flat(p, rb, rb_s) * rmat == p * rs for p in range(total))
            if affine:
                defer = self.defer_hint
                plan.calls.append(Call(SYM_BATCHED_DEFERRED if defer else SYM_BATCHED, 0, 0, 0, m, k, n, total, ls, rs))
                self.defer_pending = defer
                return plan
        # per-slice lowering reads memory directly: a deferred neighbour is materialised first
        if self.defer_pending:
            plan.flush_first = True
            self.defer_pending = False
        for p in range(total):
            lo, ro, oo = flat(p, lb, lb_s) * lmat, flat(p, rb, rb_s) * rmat, p * omat
            if rhs_bf16:
                sym = SYM_SINGLE if self._gpu_on() and k * n >= GPU_MIN_MACS else CPU_BF16
            else:
                sym = SYM_F32 if self._gpu_on() and m * k * n >= F32_MIN_MACS else CPU_F32
            plan.calls.append(Call(sym, lo, ro, oo, m, k, n))
        return plan


def run(plan: Plan, l: np.ndarray, r: np.ndarray, out: np.ndarray) -> list:
    """Execute the plan's GPU calls on caller-owned host arrays; return the
    calls that belong to the reference's CPU builtins (not executed here)."""
    lib = _lib.load()
    lf, rf, of = l.reshape(-1), r.reshape(-1), out.reshape(-1)
    if plan.flush_first:
        lib.dmc_matmul_bf16_gpu_flush()
    left = []
    for c in plan.calls:
        if not c.on_gpu:
            left.append(c)
            continue
        la = lf.ctypes.data + 4 * c.l_off
        ra = rf.ctypes.data + rf.itemsize * c.r_off
        oa = of.ctypes.data + 4 * c.out_off
        if c.symbol in (SYM_BATCHED, SYM_BATCHED_DEFERRED):
            getattr(lib, c.symbol)(la, ra, oa, c.m, c.k, c.n, c.batch, c.ls, c.rs)
        else:
            getattr(lib, c.symbol)(la, ra, oa, c.m, c.k, c.n)
        _lib.check()
    return left
