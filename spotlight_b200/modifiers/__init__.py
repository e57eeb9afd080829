"""Method registry of the decode path: the counterpart of the reference's
``spotlight/modifiers/__init__.py:1-44``. ``get_modifier(method)`` returns ``(None, cls)`` exactly as
the reference does, so a harness written for it (``_, cls = get_modifier(name); cls(model, save_ckp,
load_ckp, config)``) works unchanged. Only the generation methods exist here: training, evaluation
and the pass-through baselines are not part of the decode-time retrieval path."""


def get_modifier(method: str, model_type: str = None):
    if method == "spotlight-generation":
        from .spotlight_generation import Spotlight
        return None, Spotlight
    if method == "linearhashing-generation":
        from .linearhashing_generation import LinearHashing
        return None, LinearHashing
    if method == "upperbound-generation":
        from .upperbound_generation import UpperBound
        return None, UpperBound
    raise NotImplementedError(method, model_type)
