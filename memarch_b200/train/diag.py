"""Total diagnostics of a training run (`DIAG=1`): what a run that stalled or died without a trace would have needed.

* start-up phases: time since the start and since the previous phase, the host's resident memory / load / free RAM,
  and every visible GPU's memory (in use / peak / total);
* the same memory line every `DIAG_EVERY` steps (50);
* a kineto trace of steps `DIAG_PROF` .. `DIAG_PROF + 3` (0: none) written to `DIAG_DIR` - timings taken inside those
  steps are not measurements;
* stalls are the watchdog's job (`train.guards.Watchdog`: stacks of all threads after `WATCHDOG` seconds without a
  step); host-side time per step (data wait, enqueue, evaluation, checkpoint) is printed by the loop itself.

Without `DIAG=1` every call returns at once.  (memarch_jax/memarch_jax/diag.py:1-130 of the reference's JAX port)
"""
from __future__ import annotations

import os
import sys
import time


def host_line():
    try:
        rss = int(open("/proc/self/status").read().split("VmRSS:")[1].split()[0]) / 2 ** 20
        load = " ".join(open("/proc/loadavg").read().split()[:3])
        free = int(open("/proc/meminfo").read().split("MemAvailable:")[1].split()[0]) / 2 ** 20
        return f"host RSS {rss:.1f} GiB, load {load}, free RAM {free:.0f} GiB"
    except Exception as e:   # noqa: BLE001 - not Linux: the line is only informative
        return f"host: {e!r}"


def device_line():
    import torch
    if not torch.cuda.is_available():
        return "no GPU"
    parts = []
    for i in range(torch.cuda.device_count()):
        free, total = torch.cuda.mem_get_info(i)
        parts.append(f"{i}:{(total - free) / 2 ** 30:.1f}/{torch.cuda.max_memory_allocated(i) / 2 ** 30:.1f}/{total / 2 ** 30:.0f}")
    return "GPU GiB (in use/peak of this process/total) " + " ".join(parts)


class Diag:
    def __init__(self, env=None, out=None):
        env = os.environ if env is None else env
        self.on = env.get("DIAG") == "1"
        self.every = int(env.get("DIAG_EVERY", 50))
        self.prof_at = int(env.get("DIAG_PROF", 0))
        self.dir = env.get("DIAG_DIR", "diag")
        self.out = out or sys.stdout
        self.t0 = self.t_phase = time.time()
        self._prof = None
        if self.on:
            self._p(f"on: memory every {self.every} steps" +
                    (f"; trace of steps {self.prof_at}..{self.prof_at + 3} -> {self.dir}" if self.prof_at else ""))
            self.phase("start")

    def _p(self, *a):
        print("[diag]", *a, file=self.out, flush=True)

    def phase(self, name):
        if not self.on:
            return
        now = time.time()
        self._p(f"phase '{name}': +{now - self.t_phase:.1f} s ({now - self.t0:.1f} s since the start) | {host_line()} | {device_line()}")
        self.t_phase = now

    def step(self, i):
        """After step i - 1, before step i."""
        if not self.on:
            return
        if self.every and i % self.every == 0:
            self._p(f"step {i}: {device_line()} | {host_line()}")
        if self.prof_at and i == self.prof_at and self._prof is None:
            import torch
            acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            self._prof = torch.profiler.profile(activities=acts)
            self._prof.__enter__()
            self._p(f"trace: started at step {i}")
        elif self._prof is not None and i >= self.prof_at + 3:
            self.close()

    def close(self):
        if self._prof is not None:
            prof, self._prof = self._prof, None
            prof.__exit__(None, None, None)
            os.makedirs(self.dir, exist_ok=True)
            path = os.path.join(self.dir, f"trace_step{self.prof_at}.json")
            prof.export_chrome_trace(path)
            self._p(f"trace: written to {path}")
