"""Architectures. Importing this package registers them with ``config.registry``.

``presets/`` holds config.json files of known sizes of these architectures (no weights): what ``--random NAME`` of the
command lines and the benchmark build random models from.
"""
import json
import os

from . import qwen2  # noqa: F401

PRESET_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def preset_names():
    return sorted(f[:-5] for f in os.listdir(PRESET_DIR) if f.endswith(".json"))


def load_preset(spec: str) -> dict:
    """A raw config.json dictionary from a preset's name, a path to a config.json (or to a folder that holds one),
    or an inline JSON object."""
    spec = spec.strip()
    if spec.startswith("{"):
        return json.loads(spec)
    for path in (os.path.join(PRESET_DIR, spec + ".json"), spec, os.path.join(spec, "config.json")):
        if os.path.isfile(path):
            with open(path, "r", encoding="utf-8") as f:
                return json.load(f)
    raise ValueError(f"no preset, config.json or JSON object {spec!r}; presets: {', '.join(preset_names())}")
