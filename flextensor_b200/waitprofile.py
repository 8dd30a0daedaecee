"""Where the roles of the tensor-core GEMM kernel wait: ``python -m flextensor_b200.waitprofile``.

Needs the diagnostic build of the library (``python -m flextensor_b200.build --profile-waits``),
which this module selects by itself.  It runs the batched bf16 GEMM (``--batch`` items of
``--size``^3) with the given knob sets and prints, per knob set, the time of a launch and the SM
cycles each role of a CTA spent inside its barrier waits, per K block of the main loop:

  producer_wait_empty      the TMA producer waiting for a free pipeline stage
  issuer_wait_full         the MMA issuer waiting for a stage to land
  issuer_wait_tmem_free    the MMA issuer waiting for the epilogue to hand an accumulator back
  epilogue_wait_tmem_full  the epilogue waiting for an accumulator to complete

``--diag`` adds runs whose results are garbage but whose timings separate the bounds: 1 = stages
are signalled without being loaded (tensor pipe + epilogue only), 2 = stages are released without
MMAs (loads only), 4 = MMAs back to back with no producer and no stage hand-off (the tensor
pipe's own rate), 12 = the same with M = 64 instructions (single-CTA tiles), 20 / 36 = consecutive
MMAs go to two / four accumulators in turn (36: tiles of at most 64 columns), 68 = a second thread
issues the same MMAs at the same time (single-CTA tiles of at most 128 columns).
"""
import argparse
import json
import os
import sys


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--size", type=int, default=2048)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--knobs", action="append", default=[],
                    help="JSON knob set (repeatable); default: the 256x512 and 256x256 pair tiles")
    ap.add_argument("--diag", type=int, nargs="*", default=[0], help="diagnostic modes to run each knob set in")
    args = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    os.environ.setdefault("FTB200_LIBRARY", os.path.join(here, "lib", "libftb200_prof.so"))
    if not os.path.exists(os.environ["FTB200_LIBRARY"]):
        from . import build
        build.build_profile_waits()
    import torch
    from . import backend as B
    knob_sets = [json.loads(k) for k in args.knobs] or [
        {"cluster": 2, "tile_n": 512, "raster": 3, "group_m": 8},
        {"cluster": 2, "tile_n": 256, "raster": 3, "group_m": 4},
    ]
    n = args.size
    a = (torch.randn(args.batch, n, n, device="cuda") * 0.02).bfloat16()
    b = (torch.randn(args.batch, n, n, device="cuda") * 0.02).bfloat16()
    c = torch.empty(args.batch, n, n, device="cuda", dtype=torch.bfloat16)
    status = B.new_status()
    for knobs in knob_sets:
        for diag in args.diag:
            cfg = dict(knobs)
            if diag:
                cfg["_diag"] = diag
            for _ in range(3):
                B.bgemm_bf16(a, b, c, cfg=cfg, status=status)
            torch.cuda.synchronize()
            B.wait_profile(reset=True)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.reps):
                B.bgemm_bf16(a, b, c, cfg=cfg, status=status)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.reps
            prof = B.wait_profile(reset=True)
            ctas = max(prof["ctas"], 1)
            # K blocks one producer walks per launch: tiles per tile-walking unit x K blocks per tile
            tile_m = 256 if knobs.get("cluster", 1) == 2 else 128
            tiles = args.batch * ((n + tile_m - 1) // tile_m) * ((n + knobs["tile_n"] - 1) // knobs["tile_n"])
            units = ctas / args.reps / (2 if knobs.get("cluster", 1) == 2 else 1)
            kb_per_unit = tiles / units * (n // 64)
            per_cta = {k: v / ctas for k, v in prof.items() if k != "ctas"}
            issuers = 0.5 if knobs.get("cluster", 1) == 2 else 1.0  # only the leader CTA of a pair issues
            row = {
                "knobs": cfg, "ms": round(ms, 4), "tflops": round(args.batch * 2.0 * n ** 3 / ms / 1e9, 1),
                "status": int(status.item()),
                "sm_mhz_from_cycles": round(per_cta["epilogue_loop"] / (ms * 1e3), 0),
                "cycles_per_k_block": round(per_cta["epilogue_loop"] / kb_per_unit, 1),
                "per_k_block": {
                    "producer_wait_empty": round(per_cta["producer_wait_empty"] / kb_per_unit, 1),
                    "issuer_wait_full": round(per_cta["issuer_wait_full"] / issuers / kb_per_unit, 1),
                    "issuer_wait_tmem_free": round(per_cta["issuer_wait_tmem_free"] / issuers / kb_per_unit, 1),
                    "epilogue_wait_tmem_full": round(per_cta["epilogue_wait_tmem_full"] / kb_per_unit, 1),
                },
                "epilogue_cycles_per_tile": {
                    "tmem_ld": round(per_cta["epilogue_tmem_ld"] / (tiles / units), 0),
                    "bulk_wait": round(per_cta["epilogue_bulk_wait"] / (tiles / units), 0),
                    "convert_and_stage": round(per_cta["epilogue_stage"] / (tiles / units), 0),
                    "store_issue": round(per_cta["epilogue_store_issue"] / (tiles / units), 0),
                    "hand_back_pack_vote": round(per_cta["epilogue_vote"] / (tiles / units), 0),
                    "busy_total": round((per_cta["epilogue_loop"] - per_cta["epilogue_wait_tmem_full"]) / (tiles / units), 0),
                },
            }
            print(json.dumps(row), flush=True)


if __name__ == "__main__":
    sys.exit(main())
