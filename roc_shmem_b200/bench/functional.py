"""Functional test driver of the device API: one program, one test type per run (or all of them), a sweep of message
sizes doubling up to ``-s``, and per size: verification of the moved bytes plus average latency, bandwidth and message
rate.

    python -m torch.distributed.run --nproc-per-node 2 -m roc_shmem_b200.bench.functional -a put -s 1048576 -w 8 -z 256
    python -m roc_shmem_b200.bench.functional --list
    python -m torch.distributed.run --nproc-per-node 2 -m roc_shmem_b200.bench.functional --all --out sweep.json

Protocol per size (the reference's ``Tester::execute``, clients/functional_tests/tester.cpp:494-564): reset buffers →
barrier → launch the test kernel on the PEs that drive it → synchronize → barrier → verify → print.  Latency and
message rate come from the kernel's own timers (one per work-group, average taken), bandwidth from CUDA events around
the launch (tester.cpp:588-616).  Loop counts follow tester_arguments.hpp:71-74: 100 timed + 10 untimed iterations, 25
above 32 KiB.  The type numbers are the reference's ``-a`` values (tester.hpp:34-87); type 52, put-with-signal, is new.
Only PE 0 launches, except the collectives, the barriers, ping-pong and put-with-signal (tester.cpp:566-586).  With a
single PE every operation targets the PE itself.  The kernels live in csrc/cuda/functional_tester.cu.
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass

import torch

import roc_shmem_b200 as shmem


@dataclass(frozen=True)
class Spec:
    id: int
    name: str
    family: str          # rma | swarm | coll | amo | init | pingpong | random | sync | ptr | pg | mr | infra | put_signal
    put: bool = False
    scope: str = "thread"
    team_ctx: bool = False
    both_launch: bool = False


_S = Spec
SPECS = [
    _S(0, "get", "rma"), _S(1, "get_nbi", "rma"), _S(2, "put", "rma", put=True), _S(3, "put_nbi", "rma", put=True),
    _S(4, "get_swarm", "swarm"), _S(5, "reduction", "coll", both_launch=True),
    _S(6, "amo_fadd", "amo"), _S(7, "amo_finc", "amo"), _S(8, "amo_fetch", "amo"), _S(9, "amo_fcswap", "amo"),
    _S(10, "amo_add", "amo"), _S(11, "amo_inc", "amo"), _S(12, "amo_cswap", "amo"), _S(13, "init", "init"),
    _S(14, "ping_pong", "pingpong", both_launch=True), _S(16, "random_access", "random", put=True),
    _S(17, "barrier_all", "sync", both_launch=True), _S(18, "sync_all", "sync", both_launch=True),
    _S(19, "sync", "sync", team_ctx=True, both_launch=True), _S(20, "broadcast", "coll", both_launch=True),
    _S(21, "collect", "coll", both_launch=True), _S(22, "fcollect", "coll", both_launch=True),
    _S(23, "alltoall", "coll", both_launch=True), _S(24, "alltoalls", "coll", both_launch=True),
    _S(25, "shmem_ptr", "ptr"), _S(26, "p", "pg", put=True), _S(27, "g", "pg"),
    _S(28, "wg_get", "rma", scope="block"), _S(29, "wg_get_nbi", "rma", scope="block"),
    _S(30, "wg_put", "rma", put=True, scope="block"), _S(31, "wg_put_nbi", "rma", put=True, scope="block"),
    _S(32, "wave_get", "rma", scope="warp"), _S(33, "wave_get_nbi", "rma", scope="warp"),
    _S(34, "wave_put", "rma", put=True, scope="warp"), _S(35, "wave_put_nbi", "rma", put=True, scope="warp"),
    _S(36, "team_broadcast", "coll", team_ctx=True, both_launch=True),
    _S(37, "team_reduction", "coll", team_ctx=True, both_launch=True),
    _S(38, "team_ctx_get", "rma", team_ctx=True), _S(39, "team_ctx_get_nbi", "rma", team_ctx=True),
    _S(40, "team_ctx_put", "rma", put=True, team_ctx=True), _S(41, "team_ctx_put_nbi", "rma", put=True, team_ctx=True),
    _S(42, "team_ctx_infra", "infra", team_ctx=True), _S(43, "put_nbi_mr", "mr", put=True),
    _S(44, "amo_set", "amo"), _S(45, "amo_swap", "amo"), _S(46, "amo_fetch_and", "amo"), _S(47, "amo_fetch_or", "amo"),
    _S(48, "amo_fetch_xor", "amo"), _S(49, "amo_and", "amo"), _S(50, "amo_or", "amo"), _S(51, "amo_xor", "amo"),
    _S(52, "put_signal", "put_signal", put=True, scope="block", both_launch=True),
]
BY_ID = {s.id: s for s in SPECS}
BY_NAME = {s.name: s for s in SPECS}

_AMO_INIT = {6: 0, 7: 0, 8: 7, 9: 0, 10: 0, 11: 0, 12: 0, 44: 0, 45: 0, 46: 0xFF, 47: 0, 48: 0, 49: 0xFF, 50: 0, 51: 0}
_COLL_KIND = {5: "reduce", 37: "reduce", 20: "bcast", 36: "bcast", 21: "fcollect", 22: "fcollect", 23: "alltoall", 24: "alltoall"}


def lookup(algo: str) -> Spec:
    if algo.lstrip("-").isdigit():
        if int(algo) not in BY_ID:
            raise SystemExit(f"unknown test type {algo} (see --list)")
        return BY_ID[int(algo)]
    if algo not in BY_NAME:
        raise SystemExit(f"unknown test type {algo!r} (see --list)")
    return BY_NAME[algo]


class Tester:
    """Buffers and the per-size protocol.  Construction allocates symmetric memory: every PE must build it."""

    __test__ = False      # not a pytest class, whatever its name says

    def __init__(self, rt, max_size: int, wgs: int, wg_size: int, loop: int = 100, skip: int = 10, loop_large: int = 25,
                 large: int = 32768, ctx_options: int = 0):
        self.rt, self.max_size, self.wgs, self.wg_size = rt, max_size, wgs, wg_size
        self.loop, self.skip, self.loop_large, self.large, self.ctx_options = loop, skip, loop_large, large, ctx_options
        self.me, self.n = rt.my_pe, rt.n_pes
        self.peer = 1 if self.n > 1 else 0
        dev = rt.device
        self.n_bins = 256
        span = max(max_size * max(wgs, self.n, 1), 4096)
        span = max(span, min(max_size, 4096) * max(wgs * wg_size, self.n_bins))   # swarm slices, random bins (small sizes only)
        self.span = span
        self.sym_a = rt.zeros((span,), torch.uint8)
        self.sym_b = rt.zeros((span,), torch.uint8)
        self.local = torch.zeros(span, dtype=torch.uint8, device=dev)
        self.n_words = 128 + wgs * wg_size + wgs
        self.words = rt.zeros((self.n_words,), torch.int64)
        self.timers = torch.zeros(max(wgs, 1), dtype=torch.int64, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        g = torch.Generator(device="cpu").manual_seed(1234)
        self.pattern = torch.randint(1, 256, (span,), dtype=torch.uint8, generator=g).to(dev)    # never zero
        self.team = rt.team_world.split_strided(0, 1, self.n)      # a second team of every PE, for the team-context types
        rt.barrier_all()

    def close(self) -> None:
        self.rt.barrier_all()
        self.team.destroy()

    # ------------------------------------------------------------------------------------------------------------
    def sizes(self, spec: Spec, min_size: int, max_size: int) -> list[int]:
        if spec.family in ("amo", "pingpong", "sync", "ptr", "init", "infra"):
            return [8]
        if spec.family == "pg":
            return [s for s in (1, 2, 4, 8) if min_size <= s <= max(max_size, 1)] or [8]
        lo, hi = max(min_size, 1), max_size
        if spec.family == "coll":
            lo = max(lo, 4)
            hi = min(hi, self.span // max(self.n, 1))
        if spec.family in ("swarm", "random"):
            hi = min(hi, 4096)
        out, s = [], lo
        while s <= hi:
            out.append(s)
            s <<= 1
        return out or [lo]

    def _msgs_per_iter(self, spec: Spec) -> int:
        if spec.family in ("amo", "swarm", "random"):
            return self.wgs * self.wg_size
        if spec.family == "mr":
            return self.wgs * 64
        if spec.family == "coll":
            return 1
        return self.wgs

    def run_size(self, spec: Spec, size: int) -> dict:
        rt, me, n, peer = self.rt, self.me, self.n, self.peer
        loops = self.loop_large if size > self.large else self.loop
        skip = self.skip
        wgs, wg_size = self.wgs, self.wg_size
        if spec.family == "coll":
            wgs, wg_size = 1, min(wg_size, 256)
        total = loops + skip
        # ---- reset ----
        self.sym_a.zero_(); self.sym_b.zero_(); self.local.zero_(); self.words.zero_(); self.timers.zero_(); self.status.zero_()
        nbytes = size * wgs
        if spec.family in ("rma", "mr", "put_signal"):
            if spec.put:
                self.local[:nbytes] = self.pattern[:nbytes]
            else:
                self.sym_a[:nbytes] = self.pattern[:nbytes]
        elif spec.family == "swarm":
            nbytes = size * wgs * wg_size
            self.sym_a[:nbytes] = self.pattern[:nbytes]
        elif spec.family == "random":
            self.local[: self.n_bins * size] = self.pattern[: self.n_bins * size]
        elif spec.family == "pg":
            if not spec.put:
                self.sym_a[: 8 * wgs] = self.pattern[: 8 * wgs]
        elif spec.family == "amo":
            self.words[0] = _AMO_INIT[spec.id]
        elif spec.family == "coll":
            kind = _COLL_KIND[spec.id]
            ne = size // 4
            a32 = self.sym_a.view(torch.int32)
            if kind == "reduce":
                self.sym_a.view(torch.float32)[:ne] = 1.0
            elif kind == "bcast":
                a32[:ne] = torch.arange(ne, dtype=torch.int32, device=rt.device) + 77
            elif kind == "fcollect":
                a32[:ne] = torch.arange(ne, dtype=torch.int32, device=rt.device) + (me << 16)
            else:
                for j in range(n):
                    a32[j * ne:(j + 1) * ne] = (me << 16) + j
        torch.cuda.synchronize()
        rt.barrier_all()
        # ---- launch ----
        launches = me == 0 or spec.both_launch
        if spec.family in ("pingpong", "put_signal"):
            launches = me in (0, peer)          # a pair of PEs; the others only take part in the barriers
        team = self.team if spec.team_ctx else None
        ms = 0.0
        infra_ok = True
        if spec.family == "infra":
            infra_ok = self._team_infra()
        if launches:
            tgt = peer if me == 0 else 0
            if spec.family in ("coll", "sync"):
                tgt = 0
            ms = rt.functional_run(spec.id, size=size, wgs=wgs, wg_size=wg_size, loops=loops, skip=skip, peer=tgt, sym_a=self.sym_a,
                                   sym_b=self.sym_b, local=self.local, words=self.words, timers=self.timers, status=self.status,
                                   team=team, ctx_options=self.ctx_options, initiator=(me == 0), n_bins=self.n_bins)
        torch.cuda.synchronize()
        rt.barrier_all()
        # ---- verify ----
        ok = int(self.status.item()) == 0 and infra_ok
        i_am_target = me == peer
        if spec.family in ("rma", "mr", "put_signal"):
            if spec.put and i_am_target:
                ok = ok and torch.equal(self.sym_a[:nbytes], self.pattern[:nbytes])
            if not spec.put and me == 0:
                ok = ok and torch.equal(self.local[:nbytes], self.pattern[:nbytes])
            if spec.family == "put_signal" and i_am_target:
                ok = ok and bool((self.words[:wgs] == total).all())
        elif spec.family == "swarm" and me == 0:
            ok = ok and torch.equal(self.local[:nbytes], self.pattern[:nbytes])
        elif spec.family == "random" and i_am_target:
            got = self.sym_a[: self.n_bins * size].view(self.n_bins, size)
            want = self.pattern[: self.n_bins * size].view(self.n_bins, size)
            touched = (got != 0).any(dim=1)
            ok = ok and bool(touched.any()) and bool((got[touched] == want[touched]).all())
        elif spec.family == "pg":
            if spec.put and i_am_target:
                got = self.sym_a[: 8 * wgs].view(wgs, 8)[:, :size]
                want = torch.zeros_like(got)
                want[:, 0] = 0x5A
                ok = ok and torch.equal(got, want)
            if not spec.put and me == 0:
                ok = ok and torch.equal(self.local[: 8 * wgs].view(wgs, 8)[:, :size], self.pattern[: 8 * wgs].view(wgs, 8)[:, :size])
        elif spec.family == "amo" and i_am_target:
            count = total * wgs * wg_size
            w0 = int(self.words[0].item())
            own = self.words[64:64 + wgs * wg_size]
            want = {6: 2 * count, 10: 2 * count, 7: count, 11: count, 8: 7, 44: 44, 45: 45, 46: 0x0F, 49: 0x0F, 47: 0xF0, 50: 0xF0,
                    48: count & 1, 51: count & 1}
            if spec.id in (9, 12):
                ok = ok and bool((own == total).all())
            else:
                ok = ok and w0 == want[spec.id]
        elif spec.family == "pingpong":
            if n > 1 and me in (0, peer) or n == 1:
                ok = ok and bool((self.words[:wgs] == total).all())
        elif spec.family == "ptr" and i_am_target:
            ok = ok and bool((self.words[:wgs] == torch.arange(wgs, device=rt.device) + 0xC0FFEE).all())
        elif spec.family == "coll":
            kind = _COLL_KIND[spec.id]
            ne = size // 4
            b32 = self.sym_b.view(torch.int32)
            if kind == "reduce":
                ok = ok and bool((self.sym_b.view(torch.float32)[:ne] == float(n)).all())
            elif kind == "bcast":
                if me != 0:
                    ok = ok and torch.equal(b32[:ne], torch.arange(ne, dtype=torch.int32, device=rt.device) + 77)
            elif kind == "fcollect":
                for k in range(n):
                    ok = ok and torch.equal(b32[k * ne:(k + 1) * ne], torch.arange(ne, dtype=torch.int32, device=rt.device) + (k << 16))
            else:
                for k in range(n):
                    ok = ok and bool((b32[k * ne:(k + 1) * ne] == (k << 16) + me).all())
        rt.barrier_all()
        # ---- report (what PE 0 measured) ----
        msgs_iter = self._msgs_per_iter(spec)
        timer_ns = float(self.timers[:wgs].double().mean().item()) if launches else 0.0
        timed_msgs = loops * msgs_iter
        lat_us = timer_ns / 1e3 / max(loops * (64 if spec.family == "mr" else 1), 1)
        rate = timed_msgs / (timer_ns / 1e9) if timer_ns > 0 else 0.0
        bw_msgs = (loops if spec.family == "coll" else total) * msgs_iter
        bw = bw_msgs * size / (ms / 1e3) / 1e9 if ms > 0 else 0.0
        return {"size": size, "ok": bool(ok), "latency_us": lat_us, "bandwidth_GBs": bw, "msg_rate": rate, "loops": loops,
                "kernel_ms": ms}

    def _team_infra(self) -> bool:
        """Teams can be created up to the configured limit and the next request fails (the reference's
        team_ctx_infra_tester.cpp:100-121 expects the same of its 40-team table)."""
        rt = self.rt
        made = []
        failed_cleanly = False
        for _ in range(64):
            try:
                made.append(rt.team_world.split_strided(0, 1, self.n))
            except shmem.ShmemError:
                failed_cleanly = True
                break
        for t in made:
            t.destroy()
        return failed_cleanly and len(made) >= 1

    def run(self, spec: Spec, min_size: int = 1, max_size: int | None = None, verbose: bool = True) -> dict:
        rows = [self.run_size(spec, s) for s in self.sizes(spec, min_size, self.max_size if max_size is None else max_size)]
        oks = self.rt.bootstrap.allgather(all(r["ok"] for r in rows), tag=f"ft-{spec.id}") if self.n > 1 else [all(r["ok"] for r in rows)]
        res = {"type": spec.id, "name": spec.name, "ok": all(oks), "wgs": self.wgs, "wg_size": self.wg_size, "rows": rows}
        if verbose and self.me == 0:
            print(f"*** {spec.name} (type {spec.id}) ***")
            for r in rows:
                print(f"\n##### Message Size {r['size']} #####")
                print(f"{'Latency AVG (us)':>21}{'Bandwidth (GB/s)':>21}{'Avg Message rate (Messages/s)':>32}")
                print(f"{r['latency_us']:>21.2f}{r['bandwidth_GBs']:>21.2f}{r['msg_rate']:>32.2f}")
            print(f"{'PASS' if res['ok'] else 'FAIL'}: {spec.name}", flush=True)
        return res


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-a", "--algo", default="put", help="test type: number or name (--list)")
    ap.add_argument("-s", "--max-size", type=int, default=0, help="largest message in bytes (default 1 MiB; 64 KiB with --all)")
    ap.add_argument("--min-size", type=int, default=1)
    ap.add_argument("-w", "--wgs", type=int, default=1, help="work-groups (CTAs)")
    ap.add_argument("-z", "--wg-size", type=int, default=64, help="threads per work-group")
    ap.add_argument("-x", "--ctx", type=int, default=shmem.CTX_WG_PRIVATE, help="context option bits (1 nostore, 2 serialized, 4 wg-private, 8 shared)")
    ap.add_argument("--loop", type=int, default=100)
    ap.add_argument("--skip", type=int, default=10)
    ap.add_argument("--loop-large", type=int, default=25)
    ap.add_argument("--large", type=int, default=32768, help="messages above this many bytes use --loop-large")
    ap.add_argument("--all", action="store_true", help="run every test type (sizes capped at 64 KiB unless -s is given)")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if args.list:
        for s in SPECS:
            print(f"{s.id:3d}  {s.name}")
        return
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    specs = SPECS if args.all else [lookup(args.algo)]
    max_size = args.max_size or ((64 << 10) if args.all else (1 << 20))
    span = max(max_size * max(args.wgs, int(os.environ.get("WORLD_SIZE", 1))), 4096 * max(args.wgs * args.wg_size, 256))
    rt = shmem.init("device", device=local, heap_bytes=2 * span + (64 << 20))
    t = Tester(rt, max_size, args.wgs, args.wg_size, args.loop, args.skip, args.loop_large, args.large, args.ctx)
    results = [t.run(s, args.min_size) for s in specs]
    t.close()
    if rt.my_pe == 0:
        failed = [r["name"] for r in results if not r["ok"]]
        print(json.dumps({"n_pes": rt.n_pes, "tests": len(results), "failed": failed}))
        if args.out:
            with open(args.out, "w") as f:
                json.dump({"n_pes": rt.n_pes, "results": results}, f, indent=1)
    shmem.finalize()
    if any(not r["ok"] for r in results):
        raise SystemExit(1)


if __name__ == "__main__":
    main()
