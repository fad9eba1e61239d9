"""Makes the reference's module path resolve to the B200 implementation.

The reference instantiates its attention layers from Hydra `_target_` strings,
`src.models.attention.sblocal_attention.SBLocalAttention`
(configs/model/t2tattn_cfg/sblocal.yaml:3, configs/model/attn_cfg/sblocal.yaml:1).
`install()` registers a module of that dotted name whose `SBLocalAttention` is
`fly_b200.SBLocalAttention`, so `model/t2tattn_cfg=sblocal` and the T2T-ViT
wiring (src/models/modules/token_transformer.py:36-37,54) run unchanged.  Call
it before the model is built.  Nothing else of the reference is touched.
"""
import importlib
import sys
import types

TARGET = 'src.models.attention.sblocal_attention'


def install():
    from . import sblocal_attention as ours
    from . import masking
    parts = TARGET.split('.')
    # make sure the parent packages exist (the reference's, when it is on sys.path; stubs otherwise)
    for i in range(1, len(parts)):
        name = '.'.join(parts[:i])
        if name in sys.modules:
            continue
        try:
            importlib.import_module(name)
        except ImportError:
            pkg = types.ModuleType(name)
            pkg.__path__ = []
            sys.modules[name] = pkg
    mod = types.ModuleType(TARGET)
    mod.SBLocalAttention = ours.SBLocalAttention
    mod.FullMask, mod.LengthMask = masking.FullMask, masking.LengthMask
    mod.__doc__ = 'B200 drop-in installed by fly_b200.dropin.install()'
    sys.modules[TARGET] = mod
    parent = sys.modules['.'.join(parts[:-1])]
    setattr(parent, parts[-1], mod)
    return mod
