"""Device-side harness around the C ABI: buffers live in torch CUDA tensors, every compute call goes through
``libfkb.so``.  torch is plumbing here (allocation, streams, host<->device copies); it computes nothing.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import abi


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("fusedkernellibrary_b200 needs a CUDA device (there is no CPU fallback)")


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class DeviceWorkload:
    """A Workload whose sources and outputs are resident on the current CUDA device."""

    def __init__(self, wl, poison: int | None = 0xCD):
        _require_cuda()
        self.wl = wl
        self.lib = abi.load()
        self.src = [torch.from_numpy(s).cuda() for s in wl.sources]
        if poison is None:
            self.out = [torch.empty(n, dtype=torch.uint8, device="cuda") for n in wl.out_sizes]
        else:
            self.out = [torch.full((n,), poison, dtype=torch.uint8, device="cuda") for n in wl.out_sizes]
        self.chains = wl.chain_array()
        self.planes = wl.bind([t.data_ptr() for t in self.src], [t.data_ptr() for t in self.out])
        self.n_planes = len(wl.planes)
        self._plan = None

    def launch(self) -> None:
        """One fused launch through fkb_launch_transform / fkb_launch_divergent on the current stream."""
        if len(self.wl.chains) == 1:
            rc = self.lib.fkb_launch_transform(self.chains, self.planes, self.n_planes, current_stream_ptr())
        else:
            rc = self.lib.fkb_launch_divergent(self.chains, len(self.wl.chains), self.planes, self.n_planes, current_stream_ptr())
        abi.check(rc)

    def plan(self):
        if self._plan is None:
            p = C.c_void_p()
            abi.check(self.lib.fkb_plan_create(self.chains, len(self.wl.chains), self.planes, self.n_planes, C.byref(p)))
            self._plan = p
        return self._plan

    def launch_plan(self) -> None:
        abi.check(self.lib.fkb_plan_launch(self.plan(), current_stream_ptr()))

    def kernel_launches(self) -> int:
        return int(self.lib.fkb_plan_kernel_launches(self.plan()))

    def results(self):
        torch.cuda.synchronize()
        abi.check(self.lib.fkb_device_status())
        return [t.cpu().numpy() for t in self.out]

    def close(self) -> None:
        if self._plan is not None:
            self.lib.fkb_plan_destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def run_on_device(wl, use_plan: bool = False):
    """Uploads, launches once, downloads.  Returns one uint8 numpy array per output buffer."""
    dw = DeviceWorkload(wl)
    try:
        if use_plan:
            dw.launch_plan()
        else:
            dw.launch()
        return dw.results()
    finally:
        dw.close()


def compare(got: np.ndarray, want: np.ndarray, dst_format: int, u8_lsb: int = 0, f32_rel: float = 0.0):
    """Mismatch statistics between two output buffers.  Tolerances default to bit-exact."""
    if dst_format == abi.PIX_F32C3:
        g, w = got.view(np.float32), want.view(np.float32)
        exact = g.view(np.uint32) == w.view(np.uint32)
        bad = ~exact
        if f32_rel > 0 and bad.any():
            rel = np.abs(g[bad].astype(np.float64) - w[bad]) / np.maximum(np.abs(w[bad].astype(np.float64)), 1e-30)
            n_bad = int((rel > f32_rel).sum())
            return {"mismatch": n_bad, "max_rel": float(rel.max())}
        return {"mismatch": int(bad.sum()), "max_rel": 0.0}
    d = np.abs(got.astype(np.int16) - want.astype(np.int16))
    return {"mismatch": int((d > u8_lsb).sum()), "max_abs": int(d.max()) if d.size else 0}
