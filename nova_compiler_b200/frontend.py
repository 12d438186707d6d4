"""Python face of the textual front-end (nova_b200_module_* in include/nova_b200.h).

    m = Module(open("graph.mlir").read())
    print(m.plan("main"))                 # the fused call list; needs no GPU
    y, = m.run("main", x, w, b)           # torch CUDA tensors in signature order

Also a small command line, the stand-in for `nova-opt --nova-gpu-optimized-pipeline file.mlir` + a driver
(tools/nova-opt/nova-opt.cpp:75-144, driver.cpp:17-40):

    python -m nova_compiler_b200.frontend graph.mlir [--func main] [--plan-only] [--seed 1234]

which fills the arguments with seeded uniform[-1,1) data (indices: uniform over the gathered axis is not
known here, so integer arguments are zeros), runs the function and prints each result's shape and checksum.
"""
from __future__ import annotations

import argparse
import ctypes as C
from typing import List, Sequence, Tuple

from . import _lib as L

_TORCH_DT = None


def _torch_dtypes():
    global _TORCH_DT
    if _TORCH_DT is None:
        import torch
        _TORCH_DT = {L.F32: torch.float32, L.F16: torch.float16, L.BF16: torch.bfloat16, L.I16: torch.int16,
                     L.I32: torch.int32, L.I64: torch.int64, L.I1: torch.uint8}
    return _TORCH_DT


class Module:
    def __init__(self, text: str):
        self._lib = L.load()
        self._h = C.c_void_p()
        L.check(self._lib.nova_b200_module_parse(text.encode(), C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.nova_b200_module_free(self._h)
            self._h = None

    def signature(self, func: str) -> Tuple[List[Tuple[int, Tuple[int, ...]]], List[Tuple[int, Tuple[int, ...]]]]:
        """([(dtype, shape) of each argument], [(dtype, shape) of each result])."""
        out = []
        for is_result in (0, 1):
            n = C.c_int32(0)
            L.check(self._lib.nova_b200_module_signature(self._h, func.encode(), 0, is_result, None, C.byref(n)))
            items = []
            for i in range(n.value):
                t = L.Tensor()
                L.check(self._lib.nova_b200_module_signature(self._h, func.encode(), i, is_result, C.byref(t), None))
                items.append((t.dtype, tuple(t.shape[k] for k in range(t.rank))))
            out.append(items)
        return out[0], out[1]

    def plan(self, func: str) -> str:
        buf = C.create_string_buffer(1 << 16)
        L.check(self._lib.nova_b200_module_plan(self._h, func.encode(), buf, len(buf)))
        return buf.value.decode()

    def run(self, func: str, *args):
        import torch
        dts = _torch_dtypes()
        arg_sig, res_sig = self.signature(func)
        if len(args) != len(arg_sig):
            raise L.NovaB200Error(L.ERR_INVALID_ARG, f"@{func} takes {len(arg_sig)} arguments, got {len(args)}")
        keep, targs = [], (L.Tensor * max(len(args), 1))()
        for i, (a, (dt, shape)) in enumerate(zip(args, arg_sig)):
            if not a.is_cuda:
                raise L.NovaB200Error(L.ERR_NO_DEVICE, "arguments must be CUDA tensors; there is no CPU fallback")
            a = a.contiguous()
            keep.append(a)
            if a.dtype != dts[dt] or tuple(a.shape) != shape:
                raise L.NovaB200Error(L.ERR_INVALID_ARG, f"argument {i}: expected {dts[dt]} {shape}, got {a.dtype} {tuple(a.shape)}")
            targs[i].data, targs[i].dtype, targs[i].rank = a.data_ptr(), dt, len(shape)
            for k, s in enumerate(shape):
                targs[i].shape[k] = s
        results, tres = [], (L.Tensor * max(len(res_sig), 1))()
        for i, (dt, shape) in enumerate(res_sig):
            r = torch.empty(shape, dtype=dts[dt], device=keep[0].device if keep else "cuda")
            results.append(r)
            tres[i].data, tres[i].dtype, tres[i].rank = r.data_ptr(), dt, len(shape)
            for k, s in enumerate(shape):
                tres[i].shape[k] = s
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        L.check(self._lib.nova_b200_module_run(self._h, func.encode(), targs, len(args), tres, len(res_sig), stream))
        return results


def main(argv: Sequence[str] = None) -> int:
    ap = argparse.ArgumentParser(description="run a nova/linalg function on libnova_b200")
    ap.add_argument("file")
    ap.add_argument("--func", default="main")
    ap.add_argument("--plan-only", action="store_true")
    ap.add_argument("--seed", type=int, default=1234)
    a = ap.parse_args(argv)
    m = Module(open(a.file).read())
    print(m.plan(a.func), end="")
    if a.plan_only:
        return 0
    import torch
    dts = _torch_dtypes()
    g = torch.Generator(device="cuda")
    g.manual_seed(a.seed)
    args = []
    for dt, shape in m.signature(a.func)[0]:
        if dt in (L.F32, L.F16, L.BF16):
            args.append((torch.rand(shape, device="cuda", generator=g) * 2 - 1).to(dts[dt]))
        else:
            args.append(torch.zeros(shape, device="cuda", dtype=dts[dt]))
    for i, r in enumerate(m.run(a.func, *args)):
        torch.cuda.synchronize()
        print(f"result {i}: {tuple(r.shape)} {r.dtype} sum={r.double().sum().item():.6g} [0]={r.flatten()[0].item():.6g}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
