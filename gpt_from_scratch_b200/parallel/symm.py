"""Symmetric-memory workspaces shared by the fused communication kernels (filled in by
``fused_comm``). ``reset`` drops every cached workspace (called when the parallel state
is destroyed)."""
from __future__ import annotations

_workspaces: dict = {}


def reset() -> None:
    _workspaces.clear()
