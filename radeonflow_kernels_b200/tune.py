"""Offline tuner of the FP8 GEMM plan table (tile width x split-K or stream-K per shape).

    python -m radeonflow_kernels_b200.tune [--shapes MxNxK,...] [--out plans.txt] [--emit-inc FILE] [--pair]

The B200 analogue of the reference's brute-force tuner (tuner/gemm_tuner.py:317-549 enumerates kernel
parameterisations, compiles and times each; tuner/gemm_batch.py:8-27 walks the benchmark shapes) and of
the dispatch table it regenerates (src/gemm/gemm_launcher.cpp:229-247).  The kernels here are
shape-generic, so nothing is compiled: every candidate (tile width, split-K or stream-K) is registered through
`rf_fp8_gemm_set_plan`, timed as a CUDA graph of launches that rotate over operand sets larger than L2
(3 warm-up replays, 5 timed, median; the reference template times 3 + 10 launches,
tuner/template/gemm_perf.cpp:62-81) and the fastest is written out as "m n k block_n split_k".
The file is read back with `rf_fp8_gemm_load_plans` / RF_FP8_GEMM_PLANS; `--emit-inc` writes the
built-in table compiled into the library.
"""
import argparse
import ctypes
import statistics
import sys

NK_PAIRS = [(1536, 7168), (3072, 1536), (576, 7168), (7168, 256), (7168, 2048), (4608, 7168), (7168, 2304),
            (512, 7168), (4096, 512)]
BENCHMARK_SHAPES = [(m, n, k) for m in (1024, 6144) for (n, k) in NK_PAIRS]
STREAM_K = -1       # RF_SPLIT_STREAMK of include/rf_b200.h


def candidates(m, n, k, num_sms=148, pair=False):
    """(block_n, split_k) pairs worth timing: both tile widths; split-K only while the tiles do not
    fill the SMs and every slice keeps at least two K blocks; stream-K (split_k = -1) when the tiles leave a
    ragged last wave and every SM's share is at least two K blocks."""
    kb = k // 128
    out = []
    for bn in (128, 256) + ((512,) if pair else ()):
        rows = 256 if bn == 512 else 128
        cols = 256 if bn == 512 else bn
        tiles = -(-m // rows) * -(-n // cols)
        units = num_sms // 2 if bn == 512 else num_sms
        out.append((bn, 1))
        if bn != 512 and tiles % units != 0 and min(tiles, tiles % units + units) * kb >= 2 * units:
            out.append((bn, STREAM_K))
        for s in (2, 3, 4, 6, 8):
            if tiles * (s - 1) >= units or kb // s < 2:
                break
            out.append((bn, s))
    return out


def gemm_bytes(m, n, k):
    return m * k + n * k + 4 * m * (k // 128) + 4 * ((n + 127) // 128) * (k // 128) + 2 * m * n


def time_shape(L, torch, dev, m, n, k, bn, split, cap_stream):
    """Median device time (us) of one launch with the plan (bn, split) registered for the shape."""
    from . import _lib
    _lib.check(L.rf_fp8_gemm_set_plan(m, n, k, bn, split), "rf_fp8_gemm_set_plan")
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    reps = int(min(24, max(2, -(-300e6 // gemm_bytes(m, n, k)))))
    sets = []
    for _ in range(reps):
        a = torch.randn((m, k), device=dev, generator=g).clamp_(-240, 240).to(torch.float8_e4m3fn)
        b = torch.randn((n, k), device=dev, generator=g).clamp_(-240, 240).to(torch.float8_e4m3fn)
        a_s = torch.rand((m, k // 128), device=dev, generator=g) + 0.5
        b_s = torch.rand(((n + 127) // 128, k // 128), device=dev, generator=g) + 0.5
        sets.append((a, b, a_s, b_s, torch.empty((m, n), dtype=torch.bfloat16, device=dev)))
    sptr = ctypes.c_void_p(cap_stream.cuda_stream)

    def launch_all():
        for (a, b, a_s, b_s, c) in sets:
            L.run(a.data_ptr(), b.data_ptr(), a_s.data_ptr(), b_s.data_ptr(), c.data_ptr(), m, n, k, None, sptr)

    with torch.cuda.stream(cap_stream):
        launch_all()                      # sizes the library's split-K scratch outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(cap_stream):
        with torch.cuda.graph(graph, stream=cap_stream):
            launch_all()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(5):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps)
    return statistics.median(ts)


def tune(shapes, pair=False, log=sys.stderr):
    import torch
    from . import _lib, build
    if not torch.cuda.is_available():
        raise SystemExit("tune: needs a B200; there is no CPU path")
    build.build()
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    cap_stream = torch.cuda.Stream(device=dev)
    num_sms = torch.cuda.get_device_properties(dev).multi_processor_count
    table = []
    for (m, n, k) in shapes:
        results = []
        for (bn, s) in candidates(m, n, k, num_sms, pair):
            us = time_shape(L, torch, dev, m, n, k, bn, s, cap_stream)
            results.append((us, bn, s))
            print(f"  {m}x{n}x{k} block_n={bn} split={s}: {us:.2f} us", file=log, flush=True)
        results.sort()
        us, bn, s = results[0]
        _lib.check(L.rf_fp8_gemm_set_plan(m, n, k, bn, s), "rf_fp8_gemm_set_plan")
        table.append((m, n, k, bn, s, us))
        print(f"{m}x{n}x{k}: best block_n={bn} split={s} {us:.2f} us ({2.0 * m * n * k / us / 1e6:.0f} TFLOP/s)",
              file=log, flush=True)
    return table


def write_plans(table, path):
    with open(path, "w") as f:
        f.write("# m n k block_n split_k   (us when tuned)\n")
        for (m, n, k, bn, s, us) in table:
            f.write(f"{m} {n} {k} {bn} {s}   # {us:.2f}\n")


def write_inc(table, path):
    with open(path, "w") as f:
        f.write("// {m, n, k, tile width, split-K (-1 = stream-K)}; regenerate with "
                "`python -m radeonflow_kernels_b200.tune --emit-inc`.\n")
        for (m, n, k, bn, s, us) in table:
            f.write(f"{{{m}, {n}, {k}, {bn}, {s}}},   // {us:.2f} us\n")


def parse_shapes(text):
    return [tuple(int(v) for v in item.lower().split("x")) for item in text.split(",") if item]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shapes", default="", help="MxNxK,... (default: the 18 benchmark shapes)")
    ap.add_argument("--out", default="", help="plan file to write (m n k block_n split_k per line)")
    ap.add_argument("--emit-inc", default="", help="also write the C++ include of the built-in table")
    ap.add_argument("--pair", action="store_true", help="also time the CTA-pair configuration (block_n 512)")
    args = ap.parse_args(argv)
    shapes = parse_shapes(args.shapes) if args.shapes else BENCHMARK_SHAPES
    table = tune(shapes, pair=args.pair)
    if args.out:
        write_plans(table, args.out)
    if args.emit_inc:
        write_inc(table, args.emit_inc)
    if not args.out and not args.emit_inc:
        write_plans(table, "/dev/stdout")


if __name__ == "__main__":
    main()
