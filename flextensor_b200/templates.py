"""Config -> kernel-knob templates for CUDA tasks.

In the reference a template turns an op config into TVM schedule primitives
(flextensor/templates/cuda.py:390-661, picked at flextensor/scheduler.py:799-822).  Here
the "schedule" of an op is the knob set (``struct ftb_config``) of the hand-written kernel
that serves it, so a template is a pure function from the positional config dict the
search produces to a ``{knob: value}`` dict.  The positional layout is
``space.B200_LAYOUT``.
"""
from .space import B200_LAYOUT, op_family

_SM_COUNT = {}


def sm_count(device=None):
    """SMs of the device the 'ctas' knob is a fraction of (the current CUDA device by default);
    148, a B200, where no GPU is visible (planning on a CPU-only host)."""
    try:
        import torch
        if not torch.cuda.is_available():
            return 148
        index = torch.cuda.current_device() if device is None else int(device)
        if index not in _SM_COUNT:
            _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
        return _SM_COUNT[index]
    except Exception:
        return 148


def config_to_knobs(config, op):
    """Translate one op config (``{"spatial": [[..], ..], "reduce": .., ...}``) to kernel knobs.

    Missing type keys or an empty config mean "library defaults" (what a user gets from
    ``schedule_with_config`` with ``Config([{}], None)``).
    """
    family = op_family(op)
    knobs = {}
    if family is None or not config:
        return knobs
    layout = B200_LAYOUT[family]
    for type_key, names in layout.items():
        entities = config.get(type_key) or []
        for name, entity in zip(names, entities):
            if name == "raster":
                knobs["raster"] = int(entity[0])
                if len(entity) > 1 and int(entity[1]) > 0:
                    knobs["group_m"] = int(entity[1])
            elif name == "ctas":
                eighths = int(entity[0])
                if 0 < eighths < 8:
                    knobs["ctas"] = max(2, (sm_count() * eighths // 8) & ~1)
            else:
                knobs[name] = int(entity[0])
    return knobs


def knobs_to_config(knobs, op):
    """Inverse of ``config_to_knobs`` for the knobs that are set (used to seed a search or to
    write a hand-picked knob set into a log in the reference's format)."""
    family = op_family(op)
    if family is None:
        return {}
    config = {"fuse": [], "spatial": [], "reduce": [], "reorder": [], "inline": [], "unroll": [], "merge": [],
              "special": []}
    defaults = {"tile_n": 0, "cluster": 0, "tile_h": 0, "threads": 0, "stages": 0, "split_k": 1, "release": 1}
    for type_key, names in B200_LAYOUT[family].items():
        for name in names:
            if name == "raster":
                config[type_key].append([int(knobs.get("raster", 0)), int(knobs.get("group_m", 0))])
            elif name == "ctas":
                ctas = int(knobs.get("ctas", 0))
                config[type_key].append([8 if ctas <= 0 else max(1, min(8, round(ctas * 8 / sm_count())))])
            else:
                config[type_key].append([int(knobs.get(name, defaults.get(name, 0)))])
    return config
