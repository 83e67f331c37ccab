"""Named configurations for the random-weights mode.

The reference keeps a compiled table of the checkpoints it accepts
(src/kipp_checkpoints.h:25-79).  Here a preset is data: a file
``presets/<name>.json`` holding a ``config`` object with the same keys as a
checkpoint's ``config.json`` and an ``init`` object (weight seed, standard
deviation of the matrices, jitter of the norm scales).  Nothing in the engine
reads a preset's sizes except through the typed configuration made from it.
"""
from __future__ import annotations

import json
import os

PRESET_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def preset_names() -> list[str]:
    return sorted(f[:-5] for f in os.listdir(PRESET_DIR) if f.endswith(".json"))


def load_preset(name: str) -> tuple[dict, dict]:
    """``(config.json keys, init)`` of preset ``name``; ``init`` has ``seed``,
    ``sigma`` and ``norm_jitter``."""
    path = os.path.join(PRESET_DIR, name + ".json")
    if not os.path.isfile(path):
        raise KeyError(f"unknown preset {name!r}; there are: {', '.join(preset_names())}")
    with open(path, "r", encoding="utf-8") as f:
        data = json.load(f)
    return dict(data["config"]), dict(data.get("init", {}))
