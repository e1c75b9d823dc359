"""Write ``target_profile_b200.json`` from a bench.py line, through catopt's own profile API.

    python -m catopt_b200.make_target_profile bench_line.json [catopt checkout]

The executor times bench.py measures go where catopt's cost model and autotuner read them
(catopt_core/profile.py:75-150, 471-549):

* ``op_kernel_ns["matmul"]["MxKxN"]`` — the folded-chain GEMM at every measured shape: a floor on
  the roofline price of ``linear`` / ``matmul`` ops near that shape
  (catopt_core/cost/roofline.py:269-372);
* ``measured_ns[candidate][bucket]`` — one entry per B200 executor spec, written with
  ``record_measured`` under the ``shape_bucket`` of the benchmark's inputs, which is where
  ``Autotuned(profile=...)`` looks a candidate up before it orders its attempts
  (catopt_orchestrator/autotune.py; ``corrected_price_ns``).

Needs catopt importable (source checkout as second argument, $CATOPT_SRC, or baseline/_ref).
"""
from __future__ import annotations

import glob
import json
import math
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent

#: bench.py key -> (executor spec name, total input elements of the benchmark call)
EXECUTORS = {
    "headline": ("b200_om_decayed_chunked", 3 * 16 * 32 * 8192 * 128),
    "config2_decayed_fp32": ("b200_om_decayed_chunked", 3 * 2 * 4 * 1024 * 64),
    "decayed_bf16_few_heads_B2_H8_T8192_d128": ("b200_om_decayed_chunked", 3 * 2 * 8 * 8192 * 128),
    "decayed_fp32_B16_H32_T2048_d64": ("b200_om_decayed_chunked", 3 * 16 * 32 * 2048 * 64),
    "config1_folded_chain_fp32": ("b200_linear_chain", 64 * 512),
    "folded_chain_fp32_R4096": ("b200_linear_chain", 4096 * 512),
    "folded_chain_fp32_R16384_2048x2048": ("b200_linear_chain", 16384 * 2048),
    "config3_diag_scan_bf16": ("b200_scan_all", 8 * 4096 * 1024 * 16 + 8 * 4096 * 1024),
    "config3_shared_decay_bf16": ("b200_scan_all", 2 * 8 * 4096 * 1024),
    "config3_scan_tree_final_state_fp32": ("b200_scan", 2 * 4096 * 8 * 1024 * 16),
    "config3_all_states_fp32_T1024": ("b200_scan_all", 2 * 1024 * 8 * 1024 * 16 + 8 * 1024 * 16),
    "config3_all_prefix_maps_fp32_T1024": ("b200_omd", 2 * 1024 * 8 * 1024 * 16),
    "om_causal_bf16_B1_H32_T8192_d128": ("b200_om_causal", 3 * 32 * 8192 * 128),
    "om_causal_bf16_B2_H8_T2048_d128": ("b200_om_causal", 3 * 16 * 2048 * 128),
    "om_step_decode_bf16_H32_Tk65536_d128": ("b200_om_streaming", 32 * 128 + 2 * 32 * 65536 * 128),
}
MATMUL = {"config1_folded_chain_fp32": "64x512x512", "folded_chain_fp32_R4096": "4096x512x512",
          "folded_chain_fp32_R16384_2048x2048": "16384x2048x2048"}


def _add_catopt(argv: list[str]) -> None:
    try:
        import catopt_core  # noqa: F401

        return
    except ImportError:
        pass
    root = argv[2] if len(argv) > 2 else os.environ.get("CATOPT_SRC")
    srcs = sorted(glob.glob(os.path.join(root, "packages", "*", "src"))) if root else []
    if srcs:
        sys.path[:0] = srcs
    elif (HERE.parent / "baseline" / "_ref" / "catopt_core").is_dir():
        sys.path.insert(0, str(HERE.parent / "baseline" / "_ref"))
    else:
        raise SystemExit("catopt is not importable: pass its checkout as the second argument")


def main(argv: list[str]) -> None:
    if len(argv) < 2:
        raise SystemExit(__doc__)
    _add_catopt(argv)
    from catopt_core.profile import TargetProfile, record_measured

    line = json.loads(Path(argv[1]).read_text().strip().splitlines()[-1])
    kernels = dict(line.get("kernels", {}))
    kernels["headline"] = {"us_per_step": line["ms_per_step"] * 1e3}
    old = json.loads((HERE / "target_profile_b200.json").read_text())
    matmul = {key: round(kernels[name]["us_per_step"] * 1e3) for name, key in MATMUL.items() if name in kernels}
    tf = kernels.get("folded_chain_fp32_R16384_2048x2048", {}).get("tflops", old["tflops"])
    prof = TargetProfile(
        name=old["name"], tflops=float(tf), gbps=float(line["roofline"]["peak"]), launch_us=old["launch_us"],
        device=old["device"], measured_at=line.get("measured_at", old["measured_at"]), dispatch_us=old["dispatch_us"],
        leaf_eval_us=old["leaf_eval_us"], graph_overhead_us=old["graph_overhead_us"],
        op_kernel_ns={"matmul": matmul},
        meta={"source": "catopt_b200 bench.py on one B200, CUDA events (device time per call); written by "
                        "catopt_b200.make_target_profile through catopt_core.profile.record_measured",
              "tflops_note": "fp32-accurate matmul through the 3xTF32 tcgen05 kernel, 2048 -> 2048 at R = 16384 "
                             "(fp32-equivalent FLOP/s)",
              "gbps_note": "measured device copy bandwidth of the pool's B200s (the roofline denominator)",
              "launch_us_note": "nominal; dispatch_us / leaf_eval_us / graph_overhead_us are the reference's fallbacks",
              "bucket_note": "measured_ns buckets are shape_bucket keys: cuda:0:2^ceil(log2(total input elements))"})
    for name, (cand, numel) in EXECUTORS.items():
        if name in kernels:
            bucket = f"cuda:0:2^{math.ceil(math.log2(max(numel, 1)))}"
            prof = record_measured(prof, cand, bucket, kernels[name]["us_per_step"] * 1e3)
    (HERE / "target_profile_b200.json").write_text(prof.to_json() + "\n")
    print(f"wrote {HERE / 'target_profile_b200.json'}: {len(matmul)} matmul entries, "
          f"{sum(len(v) for v in prof.measured_ns.values())} measured executor entries")


if __name__ == "__main__":
    main(sys.argv)
