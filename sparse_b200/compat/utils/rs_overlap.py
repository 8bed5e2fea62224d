"""`utils.rs_overlap` of the reference (utils/rs_overlap.py:58-497).

`BoundedRS` there monkey-patches seven methods of every block
(utils/rs_overlap.py:436-441) and reads a dozen private attributes; here the
same rules (bounded slot pool, budget min(top_m, slots // 2), one worker
thread, close-at-demand, deferred LRU commit) live in
`sparse_b200.bounded.BoundedStager`, which the blocks call through explicit
hooks instead of being patched.  This module gives it the reference's class
name and constructor shape: `BoundedRS(core, slots=4)` where `core` is anything
with `SparseContext.layer_blocks` (the module `utils.eval_core`), `install()`
and `restore()`."""
from __future__ import annotations

from sparse_b200.bounded import BoundedStager, GraphPredictor as GraphPrediction  # noqa: F401


class BoundedRS(BoundedStager):
    def __init__(self, core, *, slots: int = 4, empty_steps: int = 0):
        blocks = dict(core.SparseContext.layer_blocks)
        super().__init__(blocks, slots=slots)
        self.core = core
        self.empty_steps = int(empty_steps)
        self._installed = False

    def configure(self, *, empty_steps: int) -> None:
        self.empty_steps = int(empty_steps)

    def install(self, batch: int = 1) -> None:          # noqa: D102  (BoundedStager.install needs the decode batch)
        super().install(batch)
        self._installed = True

    def restore(self) -> None:
        if self._installed:
            self.close()
            self._installed = False
