"""Plug the B200 kernels into an importable checkout of the reference project.

The reference has one backend switch, for KDA only (``ops_kda_backend._VALID_BACKENDS``,
ops_kda_backend.py:25-35, dispatched in ``kda_forward`` 158-251); CSA / HCA and the decode caches are
bound as module globals (``ops_fused.py:37-38``, ``run_decoding.py:47-54``).  ``install()`` registers
the backend name ``"b200"`` and rebinds those globals; ``uninstall()`` restores them.  After
``install()``, ``HybridConfig(kda_backend="b200")`` (or ``KDA_BACKEND=b200`` for the runners) makes the
reference's own modules run on these kernels.
"""
from __future__ import annotations

import importlib
import sys

_saved = {}


def _try_import(name):
    try:
        return importlib.import_module(name)
    except ImportError:
        return None


def install():
    """Register backend ``"b200"`` in the reference modules that are importable.  Returns the list of
    ``module.attribute`` names that were rebound."""
    from . import csa, decoding_cache, hca, kda

    done = []
    _try_import("ops_fused")           # before any rebinding: it copies kda_forward / naive_* into its own namespace
    okb = _try_import("ops_kda_backend")
    if okb is not None and "ops_kda_backend.kda_forward" not in _saved:
        okb._VALID_BACKENDS.add("b200")
        ref_forward = okb.kda_forward
        _saved["ops_kda_backend.kda_forward"] = (okb, "kda_forward", ref_forward)

        def kda_forward(q, k, v, g, beta, *, backend="reference", **kw):
            if backend == "b200":
                return kda.kda_forward(q, k, v, g, beta, backend="b200", **kw)
            return ref_forward(q, k, v, g, beta, backend=backend, **kw)

        okb.kda_forward = kda_forward
        done.append("ops_kda_backend.kda_forward")
        # modules that did `from ops_kda_backend import kda_forward` hold their own reference to the original
        # (ops_fused.py:36, run_decoding.py:47, run_benchmark.py:44): the stack module always, the runners when
        # they are already imported (imported later, they pick up the wrapper by themselves)
        holders = [_try_import("ops_fused")] + [sys.modules.get(n) for n in ("run_decoding", "run_benchmark")]
        for mod in holders:
            if mod is not None and getattr(mod, "kda_forward", None) is ref_forward:
                _saved[f"{mod.__name__}.kda_forward"] = (mod, "kda_forward", ref_forward)
                mod.kda_forward = kda_forward
                done.append(f"{mod.__name__}.kda_forward")

    def dispatch(ref_fn, new_fn):
        def fn(H, *a, **kw):
            return new_fn(H, *a, **kw) if H.is_cuda else ref_fn(H, *a, **kw)
        fn.__wrapped__ = ref_fn
        return fn

    # the operators at their source (so that a runner imported after install() binds the dispatching version),
    # then every module that already holds its own reference to the original
    for src, attr, new in (("ops_csa", "naive_csa", csa.naive_csa), ("ops_hca", "naive_hca", hca.naive_hca)):
        srcmod = _try_import(src)
        if srcmod is None or f"{src}.{attr}" in _saved:
            continue
        ref_fn = getattr(srcmod, attr)
        wrapped = dispatch(ref_fn, new)
        holders = [srcmod, _try_import("ops_fused"), _try_import("run_decoding"), sys.modules.get("run_benchmark")]
        for mod in holders:
            if mod is not None and getattr(mod, attr, None) is ref_fn:
                key = f"{mod.__name__}.{attr}"
                _saved[key] = (mod, attr, ref_fn)
                setattr(mod, attr, wrapped)
                done.append(key)
    rd = _try_import("run_decoding")
    if rd is not None:
        for attr, new in (("CSADecodingCache", decoding_cache.CSADecodingCache),
                          ("HCADecodingCache", decoding_cache.HCADecodingCache)):
            key = f"run_decoding.{attr}"
            if hasattr(rd, attr) and key not in _saved:
                ref_cls = getattr(rd, attr)
                _saved[key] = (rd, attr, ref_cls)

                def factory(*a, _ref=ref_cls, _new=new, **kw):
                    import torch
                    dev = kw.get("device", a[-2] if len(a) >= 2 else "cpu")
                    return _new(*a, **kw) if torch.device(dev).type == "cuda" else _ref(*a, **kw)

                setattr(rd, attr, factory)
                done.append(key)
    return done


def uninstall():
    """Undo :func:`install`."""
    okb = _try_import("ops_kda_backend")
    if okb is not None:
        okb._VALID_BACKENDS.discard("b200")
    for mod, attr, val in _saved.values():
        setattr(mod, attr, val)
    _saved.clear()
