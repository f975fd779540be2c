"""`@autotune` / `@heuristics`, with the interface of newt/runtime/autotuner.py.

`Config(kwargs, num_warps=4, num_stages=1)` and `.best_config`, the cache key
(values of `key` arguments plus the dtypes of all tensor arguments, :36-52) and
the handling of `reset_to_zero` (:72-73, 89-92) are as in the reference.  One
thing is stricter: a configuration is first asked whether it *can* run
(`JITFunction.specialize` + the plan's own `check`), and one that cannot is
dropped without being launched -- the reference finds invalid configurations by
launching them and catching the failure (:76-81), which on a shared GPU can
poison the context.
"""

from ..frontend.trace import CompileError


class Config:
    def __init__(self, kwargs, num_warps=4, num_stages=1):
        self.kwargs = dict(kwargs)
        self.num_warps = num_warps
        self.num_stages = num_stages

    def all_kwargs(self):
        out = dict(self.kwargs)
        out["num_warps"] = self.num_warps
        out["num_stages"] = self.num_stages
        return out

    def __repr__(self):
        body = ", ".join(f"{k}={v}" for k, v in self.kwargs.items())
        return f"Config({body}, num_warps={self.num_warps}, num_stages={self.num_stages})"


def _busy_for(fn, seconds):
    """Keeps the device busy with `fn` for about `seconds` (bounded in calls as well)."""
    import time

    import torch

    until = time.perf_counter() + seconds
    for _ in range(100):
        for _ in range(20):
            fn()
        torch.cuda.synchronize()
        if time.perf_counter() >= until:
            break


def _bound_args(jitfn, args, kwargs):
    bound = dict(zip(jitfn.param_names, args))
    bound.update(kwargs)
    for name, default in getattr(jitfn, "defaults", {}).items():
        bound.setdefault(name, default)
    return bound


class Autotuner:
    def __init__(self, jitfn, configs, key, reset_to_zero=None, warmup=5, rep=20):
        self.jitfn = jitfn
        self.configs = list(configs)
        self.key = list(key)
        self.reset_to_zero = list(reset_to_zero or [])
        self.warmup, self.rep = warmup, rep
        self.cache = {}
        self.best_config = None
        self.timings = {}
        self.param_names = jitfn.param_names
        self.__name__ = getattr(jitfn, "__name__", "kernel")
        # where the key's parameters sit in a positional call
        self._key_at = [self.param_names.index(k) if k in self.param_names else -1
                        for k in self.key]

    def __getitem__(self, grid):
        return lambda *args, **kwargs: self._run(grid, args, kwargs)

    def _cache_key(self, bound):
        import torch

        vals = []
        for k in self.key:
            v = bound.get(k)
            vals.append(v if type(v) in (int, float, bool) or not hasattr(v, "shape")
                        else tuple(v.shape))
        vals.extend(v.dtype for v in bound.values() if isinstance(v, torch.Tensor))
        return tuple(vals)

    def _positional_key(self, args):
        """`_cache_key` of a call that gives the key's parameters and every tensor by position
        (the usual call), without building the name -> value map; None otherwise."""
        import torch

        n = len(args)
        vals = []
        for at in self._key_at:
            if not 0 <= at < n:
                return None
            v = args[at]
            vals.append(v if type(v) in (int, float, bool) or not hasattr(v, "shape")
                        else tuple(v.shape))
        vals.extend(v.dtype for v in args if isinstance(v, torch.Tensor))
        return tuple(vals)

    def _tune(self, grid, args, kwargs, bound):
        from ..testing import do_bench

        results, last_error = [], None
        warmed = False
        for cfg in self.configs:
            call_kwargs = {**kwargs, **cfg.all_kwargs()}

            def run(call_kwargs=call_kwargs):
                for name in self.reset_to_zero:
                    bound[name].zero_()
                self.jitfn[grid](*args, **call_kwargs)

            try:
                run()  # compiles; invalid configurations raise before any launch
                if not warmed:
                    # The candidates are compared with each other, so they must all be timed in
                    # the same clock state: a chip that idled takes milliseconds of work to
                    # reach its boost clock, which the first candidates of a list of short
                    # kernels would otherwise pay for (and a later, slower one would win).
                    _busy_for(run, 0.02)
                    warmed = True
                ms = do_bench(run, warmup=self.warmup, rep=self.rep)
            except (CompileError, ValueError, RuntimeError) as e:
                last_error = e
                continue
            results.append((ms, cfg, run))
        if not results:
            raise RuntimeError(f"autotune: no valid config for {self.__name__}") from last_error
        results.sort(key=lambda r: r[0])
        # A run-off between the leaders when they are close: a chip at its power cap drifts by a
        # few percent over the seconds a list of long kernels takes, which is the size of the
        # difference between the best tiles, so the order of the list would decide.  The two are
        # timed again, taking turns, and each keeps its best time.
        if len(results) > 1 and results[1][0] <= 1.03 * results[0][0]:
            best = [results[0][0], results[1][0]]
            try:
                for _ in range(2):
                    for i in (1, 0):
                        best[i] = min(best[i], do_bench(results[i][2], warmup=self.warmup, rep=self.rep))
                results[0] = (best[0],) + results[0][1:]
                results[1] = (best[1],) + results[1][1:]
                results.sort(key=lambda r: r[0])
            except (CompileError, ValueError, RuntimeError):
                pass
        results = [(ms, cfg) for ms, cfg, _ in results]
        self.timings = {repr(c): ms for ms, c in results}
        return results[0][1]

    def _run(self, grid, args, kwargs):
        import torch

        key = None
        if not any(isinstance(v, torch.Tensor) for v in kwargs.values()):
            key = self._positional_key(args)
        bound = None
        if key is None:
            bound = _bound_args(self.jitfn, args, kwargs)
            key = self._cache_key(bound)
        best = self.cache.get(key)
        if best is None:
            bound = bound or _bound_args(self.jitfn, args, kwargs)
            best = self._tune(grid, args, kwargs, bound)
            self.cache[key] = best
            for name in self.reset_to_zero:  # tuning dirtied the accumulation buffers
                bound[name].zero_()
        self.best_config = best
        chosen = best.__dict__.get("_launch_kwargs")
        if chosen is None:
            chosen = best.__dict__["_launch_kwargs"] = best.all_kwargs()
        merged = {**kwargs, **chosen} if kwargs else chosen
        direct = getattr(self.jitfn, "_run", None)     # a JITFunction: skip building the partial
        if direct is not None and not isinstance(self.jitfn, (Autotuner, Heuristics)):
            direct(grid, *args, **merged)
        else:
            self.jitfn[grid](*args, **merged)


def autotune(configs, key, reset_to_zero=None):
    return lambda jitfn: Autotuner(jitfn, configs, key, reset_to_zero)


class Heuristics:
    def __init__(self, jitfn, values):
        self.jitfn = jitfn
        self.values = dict(values)
        self.param_names = jitfn.param_names
        self.__name__ = getattr(jitfn, "__name__", "kernel")

    def __getitem__(self, grid):
        def runner(*args, **kwargs):
            bound = _bound_args(self.jitfn, args, kwargs)
            for name, fn in self.values.items():
                kwargs[name] = fn(bound)
            return self.jitfn[grid](*args, **kwargs)

        return runner


def heuristics(values):
    return lambda jitfn: Heuristics(jitfn, values)
