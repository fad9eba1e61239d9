import importlib


def _locate(path):
    module, _, name = path.rpartition('.')
    return getattr(importlib.import_module(module), name)


def instantiate(cfg, *args, _recursive_=True, **kwargs):
    cfg = dict(cfg)
    target = _locate(cfg.pop('_target_'))
    cfg.update(kwargs)
    return target(*args, **cfg)


def call(cfg, *args, **kwargs):
    return instantiate(cfg, *args, **kwargs)
