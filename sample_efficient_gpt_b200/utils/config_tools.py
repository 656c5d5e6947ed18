"""Config loading, overriding and (de)serialisation.

Behavioural parity with utils/config_tools.py:24-135 of the reference:
  * dotted-key overrides (``{"optim.lr": 1e-3}``),
  * YAML files with a top-level ``experiments:`` map selected by ``--config-key``, YAML anchors and
    merge keys, and a ``base:`` entry naming a python config module,
  * the config is stored in checkpoints as a JSON string (``Path`` -> str) and read back from a
    string or a dict,
  * run-name templates with ``{date}``, ``{time}`` and any flattened config key.
Differences: unknown keys in a *checkpoint* config are ignored with a warning (so files written by
other versions still load); unknown keys in a YAML file are an error.
"""

from __future__ import annotations

import dataclasses
import importlib
import json
import re
from datetime import datetime
from pathlib import Path
from typing import Any

import yaml

from sample_efficient_gpt_b200.config_schema import (
    Config,
    DataConfig,
    ModelConfig,
    OptimConfig,
    TrainerConfig,
    default_cfg,
)
from sample_efficient_gpt_b200.utils.logger import logger

_SECTIONS = {"data": DataConfig, "model": ModelConfig, "optim": OptimConfig, "trainer": TrainerConfig}
_CONFIG_PACKAGES = ("sample_efficient_gpt_b200.configs", "sample_efficient_gpt.configs")


def dataclass_to_nested_dict(dc) -> dict[str, Any]:
    return dataclasses.asdict(dc)


def flatten(d: dict[str, Any], prefix: str = "") -> dict[str, Any]:
    out: dict[str, Any] = {}
    for k, v in d.items():
        key = f"{prefix}.{k}" if prefix else k
        if isinstance(v, dict):
            out.update(flatten(v, key))
        else:
            out[key] = v
    return out


def set_by_dotted(cfg, dotted_key: str, value: Any):
    """Return a copy of ``cfg`` with ``a.b.c`` replaced (frozen dataclasses included)."""
    head, _, rest = dotted_key.partition(".")
    if not dataclasses.is_dataclass(cfg) or head not in {f.name for f in dataclasses.fields(cfg)}:
        raise TypeError(f"unknown config key {dotted_key!r} for {type(cfg).__name__}")
    if rest:
        value = set_by_dotted(getattr(cfg, head), rest, value)
    return dataclasses.replace(cfg, **{head: value})


def apply_overrides(cfg, overrides: dict[str, Any]):
    for k, v in overrides.items():
        cfg = set_by_dotted(cfg, k, v)
    return cfg


def _coerce(section_cls, name: str, value: Any) -> Any:
    """YAML parses ``6e-3`` as a string and tuples as lists: bring them to the schema's types."""
    ftypes = {f.name: str(f.type) for f in dataclasses.fields(section_cls)}
    t = ftypes.get(name, "")
    if isinstance(value, str) and t.startswith("float"):
        try:
            return float(value)
        except ValueError:
            return value
    if isinstance(value, list) and t.startswith("tuple"):
        return tuple(value)
    return value


def config_from_dict(config: dict[str, Any], base_cfg: Config = default_cfg, strict: bool = True) -> Config:
    cfg = base_cfg
    for sec_name, sec_cls in _SECTIONS.items():
        section = config.get(sec_name) or {}
        known = {f.name for f in dataclasses.fields(sec_cls)}
        for k, v in section.items():
            if k not in known:
                if strict:
                    raise TypeError(f"unknown config key {sec_name}.{k}")
                logger.warning(f"ignoring unknown config key {sec_name}.{k}")
                continue
            cfg = set_by_dotted(cfg, f"{sec_name}.{k}", _coerce(sec_cls, k, v))
    extra = set(config) - set(_SECTIONS) - {"project", "base"}
    if extra and strict:
        raise TypeError(f"unknown top-level config keys {sorted(extra)}")
    if "project" in config:
        cfg = dataclasses.replace(cfg, project=config["project"])
    # rebuild so that every section is a fresh object (callers mutate non-frozen sections in place)
    return Config(
        data=dataclasses.replace(cfg.data),
        model=dataclasses.replace(cfg.model),
        optim=dataclasses.replace(cfg.optim),
        trainer=dataclasses.replace(cfg.trainer),
        project=cfg.project,
    )


def save_config(cfg: Config) -> str:
    return json.dumps(dataclass_to_nested_dict(cfg), default=str)


def load_config(config_like: str | dict[str, Any]) -> Config:
    if isinstance(config_like, str):
        config_dict = json.loads(config_like)
    elif isinstance(config_like, dict):
        config_dict = config_like
    else:
        raise TypeError(f"Unsupported config type: {type(config_like)}")
    return config_from_dict(config_dict, strict=False)


def load_python_config(name: str) -> Config:
    """``name`` is a module path or the bare name of a module in the configs package."""
    candidates = [name] if "." in name else []
    candidates += [f"{pkg}.{name}" for pkg in _CONFIG_PACKAGES[:1]]
    last_err: Exception | None = None
    for mod_name in candidates:
        if mod_name.startswith(_CONFIG_PACKAGES[1]):
            mod_name = mod_name.replace(_CONFIG_PACKAGES[1], _CONFIG_PACKAGES[0], 1)
        try:
            module = importlib.import_module(mod_name)
        except ModuleNotFoundError as e:  # try the next spelling
            last_err = e
            continue
        cfg = getattr(module, "cfg", None)
        if cfg is None:
            raise ValueError(f"Config module {mod_name} does not define cfg")
        return cfg
    raise ModuleNotFoundError(f"no config module for {name!r}: {last_err}")


def load_config_from_yaml(path: str | Path, config_key: str | None = None) -> Config:
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    experiments = raw.get("experiments")
    if config_key:
        candidates = experiments if isinstance(experiments, dict) else raw
        config_dict = candidates.get(config_key)
        if config_dict is None:
            raise KeyError(f"Config '{config_key}' not found in {path}")
    else:
        if isinstance(experiments, dict):
            raise ValueError("config_key must be provided when the YAML file defines multiple experiments")
        config_dict = {k: v for k, v in raw.items() if k in _SECTIONS or k in ("project", "base")}
    if not isinstance(config_dict, dict):
        raise TypeError(f"Invalid config structure in {path}, expected a mapping")
    config_dict = dict(config_dict)
    base_name = config_dict.pop("base", raw.get("base"))
    base_cfg = load_python_config(base_name) if base_name else default_cfg
    return config_from_dict(config_dict, base_cfg=base_cfg, strict=True)


def load_cfg(config_path: str, config_key: str | None = None) -> Config:
    """YAML path (with optional key) or python config module name. Parity: train.py:51-61."""
    if str(config_path).endswith((".yaml", ".yml")):
        p = Path(config_path)
        if not p.exists():
            packaged = Path(__file__).resolve().parent.parent / "configs" / p.name
            if packaged.exists():
                p = packaged
        return load_config_from_yaml(p, config_key)
    return load_python_config(config_path)


class _Missing(dict):
    def __missing__(self, key):
        return "NA"


def render_template(template: str, cfg, extra: dict[str, Any] | None = None) -> str:
    values = _Missing(flatten(dataclass_to_nested_dict(cfg)))
    now = datetime.now()
    values["date"] = now.strftime("%m%d")
    values["time"] = now.strftime("%H%M")
    if extra:
        values.update(extra)
    # dotted keys ("{optim.lr}") are looked up whole, not as attribute access on "optim"
    return re.sub(r"\{([^{}]+)\}", lambda m: str(values[m.group(1)]), template)


def wandb_run_name(cfg: Config, extra: dict[str, Any] | None = None) -> str:
    return render_template(cfg.trainer.run_name, cfg, extra)
