"""Arrangements: how a layer's branches are wired to the residual stream.

An arrangement is a function ``run(layer, h, pending, ctx, caches) -> pending``.
``h`` is the 32-bit residual stream, updated in place; ``pending`` is the output of
the previous branch that has not been added to ``h`` yet (or ``None``), so that the
addition can be fused with the next norm, as the reference does after attention and
after the feed-forward (src/model.cu:961-968, 1006-1018).  ``layer.branches`` is the
ordered list of the layer's branches (role, part, norm before it, norm after it) and
``caches[k]`` is what branch ``k`` keeps between steps (or ``None``).

``residual``: one branch after the other, ``h += scale * post_norm(part(shift(norm(h))))`` each (a
shift, where a branch has one, blends each normed row with the row of the token before it).  With a
mixer and a feed-forward behind a norm each this is the reference's block.  A branch without
a norm hands its part the stream itself (converted to the part's compute type); a norm after
the part that offers ``add_into(h, y)`` norms the part's output and adds it to the stream in
one 32-bit kernel.

A part may offer ``forward_from_residual(h, norm, ctx[, cache]) -> bool``: it then reads
the residual stream itself, applies the given norm inside its first kernel and adds its
output into ``h`` inside its last one (the fused few-token kernels do this).  It returns
False when it cannot take the step, and the arrangement falls back to the separate norm
and the returned branch.  Parts without the method just use that path.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import register_part


def stream_as(h, dtype):
    """The 32-bit residual stream in a part's compute type (itself when that is float32)."""
    if dtype == h.dtype:
        return h
    x = torch.empty(h.shape, dtype=dtype, device=h.device)
    ops.convert_rows(h, x)
    return x


def call_part(branch, x, ctx, cache):
    """A mixer sees the step and its cache, a feed-forward only the step."""
    if branch.role == "mixer":
        return branch.part.forward(x, ctx, cache)
    return branch.part.forward(x, ctx)


@register_part("arrangement", "residual")
def run_residual(layer, h, pending, ctx, caches):
    # a copy of the stream in the compute type, left by the kernel that last added to it
    extras = getattr(ctx, "extras", None)
    lowp = extras.pop("stream_copy", None) if extras is not None else None
    for branch, cache in zip(layer.branches, caches):
        part = branch.part
        scale = float(getattr(branch, "scale", 1.0))
        if scale != 1.0 and branch.post_norm is None:
            # a residual multiplier: the part hands back what it would add, or (where it can)
            # adds alpha times it into the stream inside its last kernel; a part that reads the
            # stream itself also applies the norm in its first kernel
            if (pending is None and branch.norm is not None
                    and getattr(branch, "shift", None) is None
                    and getattr(part, "adds_scaled", False)
                    and hasattr(part, "forward_from_residual")):
                took = (part.forward_from_residual(h, branch.norm, ctx, cache, alpha=scale)
                        if branch.role == "mixer"
                        else part.forward_from_residual(h, branch.norm, ctx, alpha=scale))
                if took:
                    lowp = None
                    continue
            if branch.norm is not None and getattr(branch, "shift", None) is None:
                x = branch.norm.forward(h, pending)
            else:
                if pending is not None:
                    h.add_(pending)
                x = (branch.shift.forward(h, branch.norm, ctx, cache.shift_state)
                     if getattr(branch, "shift", None) is not None else stream_as(h, part.dtype))
            pending, lowp = None, None
            if getattr(part, "adds_scaled", False):
                if branch.role == "mixer":
                    part.forward(x, ctx, cache, into=h, alpha=scale)
                else:
                    part.forward(x, ctx, into=h, alpha=scale)
                continue
            y = call_part(branch, x, ctx, cache)
            ops.axpy_rows(h, y if y.is_contiguous() else y.contiguous(), scale)
            continue
        if (pending is None and branch.norm is not None and branch.post_norm is None
                and getattr(branch, "shift", None) is None
                and hasattr(part, "forward_from_residual")):
            took = (part.forward_from_residual(h, branch.norm, ctx, cache)
                    if branch.role == "mixer" else part.forward_from_residual(h, branch.norm, ctx))
            if took:
                lowp = None
                continue
        if getattr(branch, "shift", None) is not None:
            # norm and blend with the row of the token before, from the stream itself
            if pending is not None:
                h.add_(pending)
                pending = None
            lowp = None
            x = branch.shift.forward(h, branch.norm, ctx, cache.shift_state)
        elif branch.norm is not None:
            x = branch.norm.forward(h, pending)              # h += pending; x = norm(h)
            if pending is not None:
                lowp = None
            pending = None
        else:
            if pending is not None:
                h.add_(pending)
                pending, lowp = None, None
            # the part reads the stream itself
            x = lowp if lowp is not None and lowp.dtype == part.dtype else stream_as(h, part.dtype)
        y = call_part(branch, x, ctx, cache)
        if branch.post_norm is not None:
            if scale != 1.0:
                y = branch.post_norm.forward(y.to(h.dtype).contiguous())
                ops.axpy_rows(h, y.to(h.dtype).contiguous(), scale)
                continue
            if hasattr(branch.post_norm, "add_into"):
                # h += norm(y), 32-bit, one kernel, which also leaves the next reader's copy
                lowp = branch.post_norm.add_into(h, y, emit=True)
                continue
            y = branch.post_norm.forward(y.to(h.dtype).contiguous())
        pending = y
    if lowp is not None and pending is None and extras is not None:
        extras["stream_copy"] = lowp
    return pending


# the name the two-branch block had before blocks became lists of branches
register_part("arrangement", "prenorm")(run_residual)
