"""forge — B200-native GPTQ / SparseGPT solver engine behind the 4Bit-Forge front end.

`from forge.gptq import GPTQ` and `from forge.backend.cuda import kernels` keep the reference's names
(forge/gptq.py, forge/backend/cuda/__init__.py); forge.moe adds the layer-level batched API.

Coexistence with the reference checkout.  The reference's driver does `import forge.utils` and
`from forge.gptq import GPTQ` (quant.py:15-17).  This package replaces `forge.gptq` and `forge.backend` and has
no `forge.utils` of its own (model loading, shard I/O and dataset code are not part of the solver path), so when
a reference checkout is importable — named by the environment variable FORGE_REFERENCE_ROOT, or simply further
down sys.path — its `forge/` directory is appended to this package's search path.  Modules that exist here win;
`forge.utils` (and anything else only the reference has) resolves to the reference's files, unchanged.
"""
import os as _os
import sys as _sys


def _reference_package_dirs():
    here = _os.path.dirname(_os.path.abspath(__file__))
    roots = []
    env = _os.environ.get("FORGE_REFERENCE_ROOT")
    if env:
        roots.append(env)
    roots += [p for p in _sys.path if p]
    seen, out = set(), []
    for r in roots:
        cand = _os.path.abspath(_os.path.join(r, "forge"))
        if cand == here or cand in seen:
            continue
        seen.add(cand)
        if _os.path.isfile(_os.path.join(cand, "__init__.py")) and _os.path.isdir(_os.path.join(cand, "utils")):
            out.append(cand)
    return out


for _d in _reference_package_dirs():
    if _d not in __path__:
        __path__.append(_d)
