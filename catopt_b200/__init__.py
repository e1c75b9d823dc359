"""catopt_b200 — sm_100a executors for catopt's lowered-module hot path.

The arithmetic lives in ``libcatopt_b200.so`` (C ABI: ``include/catopt_b200.h``,
built by ``python -m catopt_b200.build``); this package is the thin host side:

* ``ops``        one function per C-ABI entry point, torch CUDA tensors in/out
* ``executors``  ``nn.Module``s with the reference's batched-executor surface
* ``verify``     the verify gate (``verify_equiv`` / ``verify_module`` / batched)
* ``sharding``   the batch x head / batch x channel / probe partition over ranks
* ``sink``       adapter into catopt's ``Sink.executors`` table (needs catopt)
* ``gen``        bindings for the ops catopt's generated-kernel tiers mint (scan and
                 decayed-contraction handlers), in place of its Triton code generation

Importing the package does not load the library; the first call does, and
raises ``B200Error`` if it is missing — there is no CPU fallback.
"""
from ._lib import B200Error  # noqa: F401

__all__ = ["B200Error"]
