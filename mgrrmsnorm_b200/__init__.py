"""mgrrmsnorm_b200: B200 (sm_100a) kernels behind the `megagemm` operator API.

Drop-in for the two hot paths of MegaGemm -- RMSNorm forward/backward and the SwiGLU MLP -- with
the reference's public names (megagemm/__init__.py:27-52):

    from mgrrmsnorm_b200 import RMSNorm, RMSNormFunction, MegaGemmTriton, MegaGemmFunction

Exports are resolved lazily, as in the reference (:31-44), so importing the package never loads the
CUDA library; the first use does, and fails loudly if it has not been built.
"""
__version__ = "0.1.0"

_EXPORTS = {
    "RMSNorm": "rmsnorm",
    "RMSNormFunction": "rmsnorm",
    "AddRMSNorm": "rmsnorm",
    "AddRMSNormFunction": "rmsnorm",
    "MegaGemmTriton": "swiglu",
    "MegaGemmFunction": "swiglu",
    "PreNormSwiGLU": "swiglu",
}


def __getattr__(name):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module '{__name__}' has no attribute '{name}'")
    import importlib

    return getattr(importlib.import_module(f".{mod}", __name__), name)


__all__ = [*_EXPORTS, "__version__"]
