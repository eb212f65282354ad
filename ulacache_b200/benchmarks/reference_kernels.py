"""Kernel-level comparison with the UNMODIFIED reference library on the same GPU.

The reference's decode benchmark needs a patched serving framework that is not
available offline, but its native kernels are reachable through its own injection
point: ``ulacache.compiler.configure_compiler(load_jit)`` (ulacache/compiler.py:42-108).
This module supplies a ``load_jit`` built on ``tvm_ffi.cpp.load_inline`` (the header-only
kernels export TVM-FFI typed functions) and then drives the reference's own Python
loaders:

* radix top-k            ``TopKKernel<false>::plan`` + ``::transform_paged``
                         (ulacache/csrc/indexer/topk_v2.cuh:1059-1300, the kernel that carries B200
                         tuning constants) against ``ulc_topk``;
* index key store        ``load_owner_index_module("quantized", ...)``
                         (ulacache/indexer/native_quantization.py:7,
                         ulacache/csrc/owner_index/fused_store_index_cache.cuh:43) against
                         ``ulc_index_key_store``;
* host <-> HBM exchange  ``exchange_host_tier`` (ulacache/cache/kernels/cpu_residency.py:244,
                         ulacache/csrc/transfer/record_exchange.cuh:56) against ``ulc_copy_records``.

Only single-GPU kernels with well-formed inputs run; the reference's cross-GPU kernels (unbounded
spins, ``trap``) are never launched.  Both arms are timed with CUDA events after warm-up, with an
L2 flush (a 256 MB write) before every timed launch.

    python -m ulacache_b200.benchmarks.reference_kernels --build-only     # no GPU needed
    python -m ulacache_b200.benchmarks.reference_kernels --out ref.json   # one B200
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.path.join(REPO, "baseline", "_ref")
BUILD = os.path.join(REPO, "baseline", "_ref_build")


def _sanitize(text: str) -> str:
    return "".join(ch if ch.isalnum() else "_" for ch in text)


def tvm_ffi_load_jit(name, *template_args, cuda_files=None, cpp_files=None, cuda_wrappers=None, cpp_wrappers=None,
                     extra_cflags=None, extra_cuda_cflags=None, extra_ldflags=None, extra_include_paths=None,
                     **_ignored):
    """The compiler service the reference expects from its host framework: include the
    named header-only sources, export each ``(name, expression)`` wrapper as a TVM-FFI typed
    function, compile for sm_100a."""
    import tvm_ffi.cpp

    os.environ.setdefault("TVM_FFI_CUDA_ARCH_LIST", "10.0a")
    lines = [f'#include "{f}"' for f in (cuda_files or [])]
    lines.append("#include <tvm/ffi/function.h>")
    lines.append("using namespace sglang;      // the wrappers name kernels and element types of this namespace unqualified")
    for export, expr in (cuda_wrappers or []):
        lines.append(f"TVM_FFI_DLL_EXPORT_TYPED_FUNC({export}, ({expr}));")
    module = _sanitize("_".join([name, *template_args]))[:96]
    flags = ["-std=c++20", "-O3", "--expt-relaxed-constexpr", "-DSGL_CUDA_ARCH=1000",
             *[f for f in (extra_cuda_cflags or []) if not f.startswith("-I")]]
    cpp = None
    if cpp_files or cpp_wrappers:
        cl = [f'#include "{f}"' for f in (cpp_files or [])] + ["#include <tvm/ffi/function.h>"]
        cl += [f"TVM_FFI_DLL_EXPORT_TYPED_FUNC({e}, ({x}));" for e, x in (cpp_wrappers or [])]
        cpp = "\n".join(cl)
    t0 = time.time()
    mod = tvm_ffi.cpp.load_inline(module, cuda_sources="\n".join(lines), cpp_sources=cpp,
                                  extra_cflags=["-std=c++20", *[f for f in (extra_cflags or []) if not f.startswith("-I")]],
                                  extra_cuda_cflags=flags, extra_ldflags=list(extra_ldflags or []),
                                  extra_include_paths=list(extra_include_paths or []),
                                  build_directory=os.path.join(BUILD, module))
    print(f"[reference] built {module} in {time.time() - t0:.1f}s", file=sys.stderr)
    return mod


class CppArgs(list):
    """Template arguments as the reference's loaders expect them from the host framework: a
    sequence that is splatted into the module name and whose ``str`` is the C++ argument list."""

    def __str__(self):
        return ", ".join(self)


def bind_reference():
    """Put the unmodified reference on the path and give it its compiler."""
    if not os.path.isdir(os.path.join(REF, "ulacache")):
        raise RuntimeError("baseline/_ref is not installed")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import ulacache.compiler as rc

    rc.configure_compiler(tvm_ffi_load_jit)
    return rc


def reference_modules():
    """Compile (or load from the in-tree build cache) the three reference modules."""
    rc = bind_reference()
    from ulacache.cache.kernels import cpu_residency as ref_res
    from ulacache.indexer.native_quantization import load_owner_index_module

    topk = rc.load_jit("ulacache_topk_v2", cuda_files=["csrc/indexer/topk_v2.cuh"],
                       cuda_wrappers=[("plan", "sglang::TopKKernel<false>::plan"),
                                      ("transform_paged", "sglang::TopKKernel<false>::transform_paged")])
    # template arguments of FusedStoreCacheIndexerKernel: key type, index type, page size, PDL, owner degree
    store = load_owner_index_module("quantized", CppArgs(["bf16_t", "int32_t", "64", "false", "1"]), request_map=False,
                                    compile_device_module=rc.load_jit)
    exchange = ref_res._exchange_module((64, 256))
    return {"topk": topk, "store": store, "exchange": exchange, "ref_res": ref_res}


class _Timer:
    def __init__(self, device):
        import torch

        self.torch = torch
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def __call__(self, fn, iters=10, warmup=3):
        """Median microseconds per call, L2 flushed before every timed call."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        out = []
        for _ in range(iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b) * 1e3)
        out.sort()
        return out[len(out) // 2]


def bench_topk(mods, timer, rows_list, ctx_list, k=2048):
    import torch
    from ..ops import topk as ours

    dev = torch.device("cuda")
    res = []
    for ctx in ctx_list:
        for rows in rows_list:
            g = torch.Generator(device=dev).manual_seed(rows * 131 + ctx)
            scores = torch.randn((rows, ctx), device=dev, generator=g, dtype=torch.float32)
            lens = torch.full((rows,), ctx, dtype=torch.int32, device=dev)
            meta = torch.zeros((rows + 1, 2), dtype=torch.int32, device=dev)
            out_ref = torch.full((rows, k), -1, dtype=torch.int32, device=dev)
            out_ours = torch.empty((rows, k), dtype=torch.int32, device=dev)

            # the reference's serving path runs the plan once per batch and the selection once per layer:
            # the plan is made here, outside the timed call
            mods["topk"].plan(lens, meta, -1)

            def ref_call():
                mods["topk"].transform_paged(scores, lens, None, out_ref, 64, meta, None, None, 0)

            def our_call():
                ours.topk(scores, k, lens, out=out_ours)

            out_hist = torch.empty_like(out_ours)

            def our_hist_call():
                ours.topk(scores, k, lens, out=out_hist, method="hist")

            ref_call(); our_call(); our_hist_call()
            torch.cuda.synchronize()
            a = torch.sort(out_ref.long(), dim=1).values
            b = torch.sort(out_ours.long(), dim=1).values
            c = torch.sort(out_hist.long(), dim=1).values
            same = bool((a == b).all()) and bool((a == c).all())
            t_ref, t_ours, t_hist = timer(ref_call), timer(our_call), timer(our_hist_call)
            res.append({"rows": rows, "ctx": ctx, "k": k, "reference_us": round(t_ref, 2), "ours_cluster_us": round(t_ours, 2),
                        "ours_hist_us": round(t_hist, 2), "speedup": round(t_ref / min(t_ours, t_hist), 3),
                        "same_selection": same})
            print(json.dumps(res[-1]), file=sys.stderr)
    return res


def bench_index_store(mods, timer, tokens_list):
    import torch
    from ..ops import records

    dev = torch.device("cuda")
    res = []
    for n in tokens_list:
        pages = (n + 63) // 64 + 1
        g = torch.Generator(device=dev).manual_seed(n)
        keys = torch.randn((n, 128), device=dev, generator=g, dtype=torch.bfloat16)
        ids = (torch.randperm(pages * 64 - 64, device=dev, generator=g)[:n] + 64).to(torch.int32)
        pool_ref = torch.zeros((pages, 8448), dtype=torch.uint8, device=dev)
        pool_ours = torch.zeros((pages, 8448), dtype=torch.uint8, device=dev)
        view = records.make_index_view(page_ptrs=[pool_ours.data_ptr()], pages_per_rank=pages, ranks=1, my_rank=0)

        def ref_call():
            mods["store"].store(keys, pool_ref, ids, 0)

        def our_call():
            records.index_key_store(view, keys, ids, owner_only=True)

        ref_call(); our_call()
        torch.cuda.synchronize()
        same = bool((pool_ref == pool_ours).all())
        t_ref, t_ours = timer(ref_call), timer(our_call)
        res.append({"tokens": n, "reference_us": round(t_ref, 2), "ours_us": round(t_ours, 2),
                    "speedup": round(t_ref / t_ours, 3), "same_bytes": same})
        print(json.dumps(res[-1]), file=sys.stderr)
    return res


def bench_exchange(mods, timer, counts, layers=1, rec_bytes=656):
    """Host -> HBM promotion of ``n`` scattered records (the copy half of a residency plan)."""
    import torch
    from ..ops import exchange as ours

    dev = torch.device("cuda")
    ref_res = mods["ref_res"]
    res = []
    for n in counts:
        slots = max(4096, 4 * n)
        g = torch.Generator().manual_seed(n)
        host = torch.randint(0, 255, (layers, slots, rec_bytes), dtype=torch.uint8, generator=g).pin_memory()
        gpu_ref = torch.zeros((layers, slots, rec_bytes), dtype=torch.uint8, device=dev)
        gpu_ours = torch.zeros_like(gpu_ref)
        src = torch.randperm(slots, generator=g)[:n].to(torch.int32)
        dst = torch.randperm(slots, generator=g)[:n].to(torch.int32)
        ws = ref_res.create_host_tier_workspace(n, dev)
        # plan rows: record, HBM slot, host source, host destination (-1 = no write-back), previous record
        plan = torch.stack([torch.arange(n, dtype=torch.int32), dst, src, torch.full((n,), -1, dtype=torch.int32),
                            torch.full((n,), -1, dtype=torch.int32)]).to(dev)
        ws.plan.copy_(plan)
        ws.counters.zero_()
        ws.counters[2] = n                       # PlanCount (ulacache/csrc/cache/directory.cuh:6)
        src_d, dst_d = src.to(dev), dst.to(dev)

        def ref_call():
            ref_res.exchange_host_tier(host, gpu_ref, ws, rec_bytes, launch=(64, 256))

        def our_call():
            ours.copy_records(host, src_d, gpu_ours, dst_d, n, rec_bytes, src_layer_stride=host.stride(0),
                              dst_layer_stride=gpu_ours.stride(0), layers=layers)

        ref_call(); our_call()
        torch.cuda.synchronize()
        same = bool((gpu_ref == gpu_ours).all())
        t_ref, t_ours = timer(ref_call), timer(our_call)
        gb = n * layers * rec_bytes / 1e9
        res.append({"records": n, "layers": layers, "reference_us": round(t_ref, 2), "ours_us": round(t_ours, 2),
                    "reference_gbs": round(gb / (t_ref * 1e-6), 1), "ours_gbs": round(gb / (t_ours * 1e-6), 1),
                    "speedup": round(t_ref / t_ours, 3), "same_bytes": same})
        print(json.dumps(res[-1]), file=sys.stderr)
    return res


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--build-only", action="store_true", help="compile the reference modules and stop (no GPU)")
    ap.add_argument("--out", default="")
    ap.add_argument("--rows", default="8,32,64,128,256")
    ap.add_argument("--ctx", default="32768,65536,131072")
    ap.add_argument("--only", default="", help="comma list of arms to run: topk, index_key_store, exchange (default all)")
    ap.add_argument("--small", action="store_true", help="one small case per kernel (first contact with a new box)")
    args = ap.parse_args(argv)
    try:
        mods = reference_modules()
    except Exception as exc:                                  # missing tvm_ffi / nvcc: say so and stop
        print(json.dumps({"reference_kernels": "unavailable", "why": repr(exc)[:400]}))
        return 0
    if args.build_only:
        print(json.dumps({"reference_kernels": "built", "modules": sorted(k for k in mods if k != "ref_res")}))
        return 0
    import torch

    timer = _Timer(torch.device("cuda"))
    rows = [8] if args.small else [int(x) for x in args.rows.split(",")]
    ctx = [32768] if args.small else [int(x) for x in args.ctx.split(",")]
    only = {x for x in args.only.split(",") if x}
    report = {"gpu": torch.cuda.get_device_name(0),
              "timing": "CUDA events, median of 10 after 3 warm-up calls, 256 MB L2 flush before each"}
    if not only or "topk" in only:
        report["topk"] = bench_topk(mods, timer, rows, ctx)
    if not only or "index_key_store" in only:
        report["index_key_store"] = bench_index_store(mods, timer, [32] if args.small else [32, 2048, 32768])
    if not only or "exchange" in only:
        report["host_to_hbm_exchange"] = bench_exchange(mods, timer, [2048] if args.small else [2048, 65536])
    text = json.dumps(report, indent=1)
    if args.out:
        with open(args.out, "w") as fh:
            fh.write(text)
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
