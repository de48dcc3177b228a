"""Arena layout: one block of device memory per executor, intermediates packed
by liveness.

The reference allocates one zero-filled array per produced tensor and never reuses
any (cuda_compiler/buffer_planner.py:25-77).  Here every intermediate gets an
offset in a single arena; two buffers may share bytes when their live ranges (in
step indices) do not overlap.  Graph outputs stay live to the end.  ``persistent``
buffers (zero padding that must survive between runs) get a private range.
"""

from __future__ import annotations

from cuda_compiler.cuda_program import BufferAllocation

ALIGN = 256


def _align(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def plan_buffers(steps, input_specs, output_specs, weight_specs, compute_dtype="float16", analysis=None):
    """Returns the list of ``BufferAllocation`` with ``offset`` filled in; the arena
    size is ``max(offset + size)`` rounded up (also stored on the analysis object)."""
    if analysis is None:
        raise ValueError("plan_buffers needs the Analysis produced by subgraph_analyzer.analyze")
    n_steps = len(steps)
    bufs: dict[str, BufferAllocation] = analysis.buffers
    seen: set[str] = set()
    for i, names in enumerate(analysis.step_tensors):
        for t in names:
            view = analysis.views.get(t)
            b = bufs.get(view.buffer) if view is not None else bufs.get(t)
            if b is None:
                continue
            if b.name not in seen:
                b.first_step = i
                seen.add(b.name)
            b.last_step = i
    for spec in output_specs:
        view = analysis.views.get(spec.name)
        if view is not None and view.buffer in bufs:
            bufs[view.buffer].last_step = n_steps
            if view.buffer not in seen:
                bufs[view.buffer].first_step = 0
                seen.add(view.buffer)

    cursor = 0
    placed: list[BufferAllocation] = []
    order = sorted((b for b in bufs.values() if b.size_bytes > 0), key=lambda b: (not b.persistent, -b.size_bytes))
    for b in order:
        if b.persistent:
            b.first_step, b.last_step = 0, n_steps
        if b.name not in seen and not b.persistent:
            b.offset = 0  # never touched by a step; harmless placeholder
            continue
        need = _align(b.size_bytes)
        conflicts = sorted((p.offset, p.offset + _align(p.size_bytes)) for p in placed
                           if not (p.last_step < b.first_step or b.last_step < p.first_step))
        at = 0
        for lo, hi in conflicts:
            if at + need <= lo:
                break
            at = max(at, hi)
        b.offset = at
        placed.append(b)
        cursor = max(cursor, at + need)
    analysis.arena_bytes = cursor
    return list(bufs.values())
