"""`@dt.kernel`: read the tile function, build its newt kernel, pick tile sizes, launch.

A `Kernel` keeps, per argument signature (ranks and dtypes), the newt kernel built from the
function (`codegen.generate` -> `JITFunction.from_ast`; no source text is executed or parsed
on the way) and, per shape bucket, the configuration a search chose for it
(`tuning.Search`, against the eager run of the same function as the oracle).  What callers see
is what deuteron/runtime.py of the reference offers: calling the kernel, `.ref` (the eager
PyTorch run), `.to_newt_source`, `.best_config`, `dt.Config`, and the environment switches
DEUTERON_INTERPRET, DEUTERON_VERBOSE and DEUTERON_CACHE_DIR.
"""

import ast
import hashlib
import inspect
import os
import textwrap

import torch

from ..frontend.trace import CompileError
from ..runtime.autotuner import _busy_for
from . import codegen, tuning
from .language import EagerTensor, eager_device
from .tuning import Config  # noqa: F401  (re-exported as dt.Config)


def _bucket(n):
    """Shapes that round up to the same power of two share a tuned configuration."""
    n = int(n)
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


class _Built:
    """One argument signature of a Kernel: the generated kernel and its jit."""

    def __init__(self, generated):
        from .. import language as nl
        import newt_b200

        self.generated = generated
        self.jit = newt_b200.runtime.jit.JITFunction.from_ast(
            generated.fndef, {"nl": nl, "newt": newt_b200, "__name__": "newt_b200.deuteron.generated"})

    @property
    def source(self):
        return self.generated.source


class Kernel:
    def __init__(self, fn, config=None, autotune=True, samples=12, verbose=False):
        self.fn = fn
        self.__name__ = fn.__name__
        self.__doc__ = fn.__doc__
        self.fndef = ast.parse(textwrap.dedent(inspect.getsource(fn))).body[0]
        self.arg_names = [a.arg for a in self.fndef.args.args]
        self.fixed_config = Config(config) if config else None
        self.autotune_enabled = autotune and config is None
        self.samples = samples
        self.verbose = verbose or bool(os.environ.get("DEUTERON_VERBOSE"))
        self._built = {}       # argument signature -> _Built
        self._chosen = {}      # tuning key -> Config
        self._last = None

    # ---- what users call ---------------------------------------------------------------------

    def __call__(self, *args):
        if os.environ.get("DEUTERON_INTERPRET"):
            return self.ref(*args)
        built = self.built_for(args)
        self.launch(built, args, self.fixed_config or self.config_for(built, args))

    def ref(self, *args):
        """The function body run as plain PyTorch on whole-dimension tiles: the oracle."""
        device = next((a.device for a in args if torch.is_tensor(a)), None)
        with eager_device(device):
            return self.fn(*[EagerTensor(a) if torch.is_tensor(a) else a for a in args])

    def to_newt_source(self, *args):
        return self.built_for(args).source

    @property
    def best_config(self):
        return self._last if self._last is not None else self.fixed_config

    # ---- building ----------------------------------------------------------------------------------

    def built_for(self, args):
        signature = tuple((a.dim(), str(a.dtype)) if torch.is_tensor(a) else type(a).__name__
                          for a in args)
        built = self._built.get(signature)
        if built is None:
            built = self._built[signature] = _Built(codegen.generate(self.fn, self.fndef, args))
            if self.verbose:
                print(f"=== deuteron: newt kernel generated for {self.__name__} ===\n{built.source}")
        return built

    # ---- launching -----------------------------------------------------------------------------------

    def launch_parts(self, built, args, config):
        """(grid, positional arguments, keyword arguments) of the newt launch under `config`."""
        gen = built.generated
        given = dict(zip(self.arg_names, args))
        extents = {}
        for kind, name in gen.params:
            if kind == "tensor":
                extents.update({f"{name}_d{d}": int(n) for d, n in enumerate(given[name].shape)})
            else:
                extents[name] = given[name]

        def length(symbol):
            return int(extents[symbol]) if symbol in extents else int(symbol)

        blocks = {axis.block: (_bucket(length(axis.size)) if axis.kind == "full" else config[axis.block])
                  for axis in gen.tile_vars}
        grid = tuple(-(-length(axis.size) // blocks[axis.block]) for axis in gen.grid_tiles)
        positional = []
        for kind, name in gen.params:
            value = given[name]
            positional.append(value)
            if kind == "tensor":
                positional += [int(n) for n in value.shape] + [int(n) for n in value.stride()]
        keywords = dict(blocks, num_warps=config.num_warps, num_stages=config.get("num_stages", 3))
        return grid, positional, keywords

    def launch(self, built, args, config):
        grid, positional, keywords = self.launch_parts(built, args, config)
        built.jit[grid](*positional, **keywords)

    # ---- configurations --------------------------------------------------------------------------------

    def tuning_key(self, built, args):
        digest = hashlib.sha256(built.source.encode()).hexdigest()[:12]
        shapes = tuple(tuple(_bucket(n) for n in a.shape) if torch.is_tensor(a) else None for a in args)
        dtypes = tuple(str(a.dtype) if torch.is_tensor(a) else "" for a in args)
        return f"{tuning.CACHE_VERSION}:{self.__name__}:{digest}:{shapes}:{dtypes}"

    def config_for(self, built, args):
        key = self.tuning_key(built, args)
        config = self._chosen.get(key)
        if config is None:
            config = tuning.ConfigFile.lookup(key)
            if config is None:
                space = tuning.search_space(built.generated.tunable, built.generated.has_dot)
                if self.autotune_enabled:
                    config = self.search(built, args, space)
                    tuning.ConfigFile.remember(key, config)
                else:
                    config = tuning.middle_of(space)
            self._chosen[key] = config
        self._last = config
        return config

    def search(self, built, args, space):
        """Times the configurations whose result matches the eager run, on copies of the
        arguments (the caller's tensors are not touched until the real launch)."""
        from ..testing import do_bench

        gen = built.generated
        names = self.arg_names

        def copies():
            return [a.clone() if torch.is_tensor(a) else a for a in args]

        oracle_args = copies()
        self.ref(*oracle_args)
        wanted = {name: dict(zip(names, oracle_args))[name] for name in gen.store_params}
        scratch = copies()
        outputs = {name: dict(zip(names, scratch))[name] for name in gen.store_params}
        pristine = {name: dict(zip(names, args))[name] for name in gen.store_params}

        def say(config, what):
            if self.verbose:
                print(f"  {dict(config)}: {what}")

        def plan_identity(config):
            _, positional, keywords = self.launch_parts(built, scratch, config)
            plan = built.jit.specialize(*positional, **keywords).plan
            describe = getattr(plan, "hardware_key", None)
            return describe() if describe else None

        clock_state = {"warm": False}

        def measure(config):
            for name, out in outputs.items():
                out.copy_(pristine[name])
            try:
                self.launch(built, scratch, config)
                torch.cuda.synchronize()
            except (CompileError, ValueError, RuntimeError) as problem:
                say(config, f"cannot run ({str(problem)[:80]})")
                return None
            for name, want in wanted.items():
                loose = gen.has_dot or want.dtype in (torch.float16, torch.bfloat16)
                bar = 2e-2 if loose else 1e-3
                if not torch.allclose(outputs[name].float(), want.float(), rtol=bar, atol=bar):
                    say(config, "differs from the eager run, dropped")
                    return None
            if not clock_state["warm"]:
                # candidates are compared with each other: all of them are timed on a chip that
                # has been busy long enough to sit at its working clock
                _busy_for(lambda: self.launch(built, scratch, config), 0.02)
                clock_state["warm"] = True
            ms = do_bench(lambda: self.launch(built, scratch, config), warmup=3, rep=10)
            say(config, f"{ms:.4f} ms")
            return ms

        best, ms = tuning.Search(space, measure, plan_identity, samples=self.samples,
                                 always=tuning.preferred(gen.tunable, gen.has_dot)).run()
        if best is None:
            raise RuntimeError(f"deuteron: no configuration of {self.__name__} both runs and matches "
                               f"its eager run (DEUTERON_VERBOSE=1 lists what was tried)")
        if self.verbose:
            print(f"deuteron: {self.__name__} -> {dict(best)} ({ms:.4f} ms)")
        return best


def kernel(fn=None, *, config=None, autotune=True, samples=12, verbose=False):
    """@dt.kernel -- a tile-language function compiled to an autotuned sm_100a kernel launch."""
    if fn is None:
        return lambda f: Kernel(f, config=config, autotune=autotune, samples=samples, verbose=verbose)
    return Kernel(fn)
