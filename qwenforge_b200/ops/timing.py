"""Per-kernel device times: CUDA events around every call that goes through `qwenforge_b200.ops`.

    with KernelTimer() as timer:
        model.step(...)
    print(timer.report())

Parts call their kernels as `ops.<name>(...)`, so the timer puts a recording wrapper in each name's place for the
time of the `with` block and puts the functions back afterwards. Events cannot time work inside a CUDA graph
capture or replay: time steps that are issued launch by launch (`cuda_graphs=False`, `--no-graphs`). The times are
those of each call alone on the stream, back to back: what overlaps across kernels (programmatic dependent launch)
shows up in the later kernel's time.
"""
from __future__ import annotations

import torch

TIMED = ("embed_gather", "gather_rows", "add_rms_norm", "residual_add", "linear", "gemm_f32", "rope_cache_write",
         "attention_generic", "attention_prefill", "attention_prefill_tc", "attention_decode", "swiglu", "skinny_gemm",
         "tc_gemm", "sample", "decode_advance")


class KernelTimer:
    def __init__(self, names=TIMED):
        self.names = tuple(names)
        self.records: list = []   # (label, start event, end event)
        self._saved: dict = {}

    def _wrap(self, name, fn):
        def timed(*args, **kwargs):
            label = name
            if name == "skinny_gemm" and args:
                label = f"skinny_gemm[{('plain', 'residual', 'swiglu', 'qkv')[args[0]]}]"
            elif name == "linear" and len(args) >= 2:
                label = f"linear[{args[0].shape[0]}x{args[1].shape[0]}x{args[1].shape[1]}]"
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = fn(*args, **kwargs)
            end.record()
            self.records.append((label, start, end))
            return out
        return timed

    def __enter__(self):
        from .. import ops
        for name in self.names:
            fn = getattr(ops, name, None)
            if fn is not None:
                self._saved[name] = fn
                setattr(ops, name, self._wrap(name, fn))
        return self

    def __exit__(self, *exc):
        from .. import ops
        for name, fn in self._saved.items():
            setattr(ops, name, fn)
        self._saved.clear()

    def totals(self) -> list:
        """(label, calls, total ms) by falling total; synchronises the device."""
        torch.cuda.synchronize()
        by_label: dict = {}
        for label, start, end in self.records:
            calls, ms = by_label.get(label, (0, 0.0))
            by_label[label] = (calls + 1, ms + start.elapsed_time(end))
        return sorted(((k, c, ms) for k, (c, ms) in by_label.items()), key=lambda r: -r[2])

    def report(self) -> str:
        rows = self.totals()
        whole = sum(ms for _, _, ms in rows) or 1.0
        lines = [f"{'kernel':<40}{'calls':>8}{'total ms':>12}{'us/call':>10}{'share':>8}"]
        for label, calls, ms in rows:
            lines.append(f"{label:<40}{calls:>8}{ms:>12.3f}{ms / calls * 1e3:>10.1f}{ms / whole:>8.1%}")
        lines.append(f"{'all':<40}{sum(c for _, c, _ in rows):>8}{whole:>12.3f}")
        return "\n".join(lines)
