"""Memory ledger: device and pinned-host allocations labelled by a scope stack ("weights", "kv",
"workspace/attention", "peer-split"), with a report of bytes per scope and a byte budget that refuses
allocations past it.  Reference: cuteafd-ffi/src/memory_ledger.rs:1-12, shared/memory/budget.rs."""
from __future__ import annotations

import contextlib
import threading
from collections import defaultdict

_state = threading.local()


class BudgetExceeded(MemoryError):
    pass


class Ledger:
    def __init__(self, budget_bytes: int | None = None):
        self.by_scope = defaultdict(int)
        self.budget = budget_bytes
        self.total = 0
        self.lock = threading.Lock()

    def _scope(self) -> str:
        return "/".join(getattr(_state, "stack", [])) or "unscoped"

    @contextlib.contextmanager
    def scope(self, name: str):
        st = getattr(_state, "stack", None)
        if st is None:
            st = _state.stack = []
        st.append(name)
        try:
            yield self
        finally:
            st.pop()

    def charge(self, nbytes: int, what: str = ""):
        with self.lock:
            if self.budget is not None and self.total + nbytes > self.budget:
                raise BudgetExceeded(f"{what or 'allocation'} of {nbytes} bytes in scope {self._scope()} exceeds the budget "
                                     f"({self.total} of {self.budget} bytes used)")
            self.by_scope[self._scope()] += nbytes
            self.total += nbytes

    def release(self, nbytes: int, scope: str):
        with self.lock:
            self.by_scope[scope] -= nbytes
            self.total -= nbytes

    def alloc(self, *shape, dtype=None, device=None, what: str = ""):
        import torch
        t = torch.zeros(*shape, dtype=dtype, device=device)
        self.charge(t.numel() * t.element_size(), what)
        return t

    def charge_tree(self, obj, what: str = ""):
        """Charge every tensor reachable from a (nested) object, e.g. a DeviceWeights."""
        import torch
        seen, total, stack = set(), 0, [obj]
        while stack:
            o = stack.pop()
            if isinstance(o, torch.Tensor):
                if o.data_ptr() not in seen:
                    seen.add(o.data_ptr())
                    total += o.numel() * o.element_size()
            elif isinstance(o, (list, tuple)):
                stack.extend(o)
            elif isinstance(o, dict):
                stack.extend(o.values())
            elif hasattr(o, "__dict__"):
                stack.extend(vars(o).values())
        self.charge(total, what)
        return total

    def report(self) -> dict:
        with self.lock:
            return {"total_bytes": self.total, "budget_bytes": self.budget,
                    "scopes": {k: v for k, v in sorted(self.by_scope.items(), key=lambda kv: -kv[1]) if v}}


LEDGER = Ledger()
