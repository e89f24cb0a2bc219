"""Named config.json files shipped with the package (the benchmark's model shapes).

They are data: each is the config.json of a model folder, read like any other.
"""
from __future__ import annotations

import json
import os
from typing import List

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def preset_names() -> List[str]:
    return sorted(f[:-5] for f in os.listdir(_DIR) if f.endswith(".json"))


def preset_config(name: str) -> dict:
    path = os.path.join(_DIR, name + ".json")
    if not os.path.isfile(path):
        raise KeyError(f"no preset {name!r} (known: {', '.join(preset_names())})")
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)
