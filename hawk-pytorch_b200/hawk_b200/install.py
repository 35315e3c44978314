"""Binds the sm_100a operators into an imported copy of the reference package.

The reference has no plugin registry; its hot-path seam is three names imported at the top of
hawk/hawk.py (hawk/hawk.py:12-14).  `install()` rebinds them, so the reference's own
HawkModel / HawkConfig then run on the kernels of this library:

    import hawk, hawk_b200.install
    hawk_b200.install.install(hawk)          # before constructing HawkModel
    model = hawk.HawkModel(cfg).cuda()

`uninstall()` restores the original bindings.
"""
from __future__ import annotations

from . import ops

_saved = {}


def install(hawk_pkg) -> None:
    mod = hawk_pkg.hawk  # the module hawk/hawk.py
    if id(mod) in _saved:
        return
    _saved[id(mod)] = (mod, mod.fused_linear_scan, mod.fused_cross_entropy, mod.Conv1D)
    mod.fused_linear_scan = ops.fused_linear_scan      # hawk/hawk.py:186
    mod.fused_cross_entropy = ops.fused_cross_entropy  # hawk/hawk.py:295-299
    mod.Conv1D = ops.Conv1D                            # hawk/hawk.py:117-120 (same .w / .b parameters)


def uninstall(hawk_pkg) -> None:
    entry = _saved.pop(id(hawk_pkg.hawk), None)
    if entry is not None:
        mod, scan, ce, conv = entry
        mod.fused_linear_scan, mod.fused_cross_entropy, mod.Conv1D = scan, ce, conv
