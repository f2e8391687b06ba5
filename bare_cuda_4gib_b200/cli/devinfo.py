"""`llm-devinfo`: the device and the memory that is left once a CUDA context exists.

    bin/llm-devinfo [--kv] [--out FILE]

Options and output follow cuongvng/bare-cuda-4gib's tool (bench/src/devinfo_main.cc:12-47,
engine/src/device_info.cpp:67-100): the long form lists the device's limits and the memory
before and after this process created its context; `--kv` prints the one-line key=value form;
`--out FILE` appends that line, with a time stamp, to a log.  Everything is read, nothing is
set.  Free memory before the context comes from NVML (a query only); where NVML is not usable
it is reported equal to the figure after.
"""

from __future__ import annotations

import argparse
import sys
import time

MIB = 1024 * 1024


def query(device: int = 0) -> dict:
    import torch

    free_before = None
    try:
        import pynvml
        pynvml.nvmlInit()
        free_before = int(pynvml.nvmlDeviceGetMemoryInfo(pynvml.nvmlDeviceGetHandleByIndex(device)).free)
        pynvml.nvmlShutdown()
    except Exception:       # no NVML here: fall back below
        free_before = None
    if not torch.cuda.is_available():
        raise SystemExit("[llm] no CUDA device")
    torch.cuda.init()
    torch.zeros(1, device=f"cuda:{device}")      # forces the context
    free_after, total = torch.cuda.mem_get_info(device)
    p = torch.cuda.get_device_properties(device)
    get = lambda name, default=0: getattr(p, name, default)
    clock_khz, bus_bits = int(get("memory_clock_rate")), int(get("memory_bus_width"))
    return {
        "device": device, "name": p.name, "cc_major": p.major, "cc_minor": p.minor, "sm_count": p.multi_processor_count,
        "warp_size": int(get("warp_size", 32)), "shared_mem_per_block": int(get("shared_memory_per_block")),
        "shared_mem_per_block_optin": int(get("shared_memory_per_block_optin")),
        "shared_mem_per_sm": int(get("shared_memory_per_multiprocessor")),
        "regs_per_sm": int(get("regs_per_multiprocessor")), "l2_cache_bytes": int(get("L2_cache_size")),
        "memory_bus_width_bits": bus_bits, "memory_clock_khz": clock_khz,
        # double data rate: two transfers per clock (device_info.h:41-44)
        "bandwidth_gbps": 2.0 * clock_khz * 1e3 * (bus_bits / 8.0) / 1e9,
        "total": int(total), "free_before": int(free_before if free_before is not None else free_after),
        "free_after": int(free_after),
    }


def format_kv(b: dict) -> str:
    overhead = max(0, b["free_before"] - b["free_after"])
    return (f'name="{b["name"]}" sm={b["cc_major"]}{b["cc_minor"]} sms={b["sm_count"]} total_mib={b["total"] // MIB} '
            f'free_pre_mib={b["free_before"] // MIB} free_post_mib={b["free_after"] // MIB} '
            f'ctx_overhead_mib={overhead // MIB} reserved_mib={(b["total"] - b["free_after"]) // MIB}')


def format_long(b: dict) -> str:
    overhead = max(0, b["free_before"] - b["free_after"])
    mib = lambda n: f"{n / MIB:.1f}"
    return "\n".join([
        f'device {b["device"]}: {b["name"]} (sm_{b["cc_major"]}{b["cc_minor"]})',
        f'  SMs                      : {b["sm_count"]}',
        f'  warp size                : {b["warp_size"]}',
        f'  shared mem / block       : {b["shared_mem_per_block"] // 1024} KiB ({b["shared_mem_per_block_optin"] // 1024} KiB opt-in)',
        f'  shared mem / SM          : {b["shared_mem_per_sm"] // 1024} KiB',
        f'  32-bit regs / SM         : {b["regs_per_sm"]}',
        f'  L2 cache                 : {b["l2_cache_bytes"] // 1024} KiB',
        f'  memory bus               : {b["memory_bus_width_bits"]} bit @ {b["memory_clock_khz"] // 1000} MHz',
        f'  theoretical bandwidth    : {b["bandwidth_gbps"]:.1f} GB/s',
        f'  VRAM total               : {mib(b["total"])} MiB',
        f'  VRAM free (pre-alloc)    : {mib(b["free_before"])} MiB',
        f'  VRAM free (post-context) : {mib(b["free_after"])} MiB',
        f'  context overhead delta   : {mib(overhead)} MiB',
        f'  total reserved (unusable): {mib(b["total"] - b["free_after"])} MiB',
        f'  => allocatable budget    : {mib(b["free_after"])} MiB',
    ]) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm-devinfo", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kv", action="store_true", help="print the one-line key=value form")
    ap.add_argument("--out", default=None, help="append the key=value line, time-stamped, to this file")
    args = ap.parse_args(argv)
    b = query(0)
    kv = format_kv(b)
    sys.stdout.write(kv + "\n" if args.kv else format_long(b))
    if args.out:
        try:
            with open(args.out, "a") as f:
                f.write(time.strftime("%Y-%m-%dT%H:%M:%S") + " " + kv + "\n")
        except OSError:
            print(f"cannot open {args.out} for writing", file=sys.stderr)
            return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
