"""A small, dependency-free composer for Hydra-style YAML config trees.

The reference drives everything through ``@hydra.main(config_path="configs",
config_name="default")`` (torchprime/torch_xla_models/train.py:29) and OmegaConf
``DictConfig`` objects.  Neither hydra nor omegaconf is a dependency here; this
module implements the part of the grammar the reference's recipes use:

* ``defaults:`` lists with ``_self_``, ``group: option``, ``override group: option``
  and bare config names (``- default``), resolved relative to the file's own
  directory, so ``model/llama-3-8b.yaml`` can pull ``sharding: llama-fsdp`` from
  ``model/sharding/llama-fsdp.yaml`` and have it land under ``model.sharding``;
* command-line overrides ``a.b.c=value``, ``group=option``, ``group/sub=option``,
  ``+new.key=value``, ``~key`` (delete), with YAML-typed values (``null``,
  ``[a,b]``, numbers, booleans);
* ``--config-name NAME`` to pick a different top-level file.

The result is a :class:`Config`: a ``dict`` subclass with attribute access that
keeps literal dotted keys (the sharding maps use parameter paths such as
``model.layers.*.mlp.up_proj.weight`` as plain keys).
"""

from __future__ import annotations

import copy
import os
from typing import Any, Iterable

import yaml

__all__ = ["Config", "compose", "parse_cli", "to_container", "load_yaml", "CONFIG_ROOT"]

CONFIG_ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")


class Config(dict):
  """Attribute-style dict.  Nested dicts are converted on the way in."""

  def __init__(self, *args, **kwargs):
    super().__init__()
    for k, v in dict(*args, **kwargs).items():
      self[k] = v

  @staticmethod
  def _wrap(v):
    if isinstance(v, Config):
      return v
    if isinstance(v, dict):
      return Config(v)
    if isinstance(v, (list, tuple)):
      return [Config._wrap(x) for x in v]
    return v

  def __setitem__(self, k, v):
    super().__setitem__(k, Config._wrap(v))

  def __getattr__(self, k):
    try:
      return self[k]
    except KeyError:
      raise AttributeError(f"config has no key '{k}' (keys: {list(self.keys())})") from None

  def __setattr__(self, k, v):
    self[k] = v

  def __delattr__(self, k):
    try:
      del self[k]
    except KeyError:
      raise AttributeError(k) from None

  def __deepcopy__(self, memo):
    return Config({k: copy.deepcopy(v, memo) for k, v in self.items()})

  def update(self, *args, **kwargs):
    for k, v in dict(*args, **kwargs).items():
      self[k] = v

  def setdefault(self, k, default=None):
    if k not in self:
      self[k] = default
    return self[k]

  def select(self, dotted: str, default=None):
    """Walk ``a.b.c`` through nested configs; literal dotted keys win over walking."""
    if dotted in self:
      return self[dotted]
    node: Any = self
    for part in dotted.split("."):
      if isinstance(node, dict) and part in node:
        node = node[part]
      else:
        return default
    return node

  def to_container(self) -> dict:
    return to_container(self)


def to_container(node):
  """Plain ``dict``/``list`` copy of a config (the analogue of ``OmegaConf.to_container``)."""
  if isinstance(node, dict):
    return {k: to_container(v) for k, v in node.items()}
  if isinstance(node, (list, tuple)):
    return [to_container(v) for v in node]
  return node


def load_yaml(path: str) -> dict:
  with open(path) as f:
    data = yaml.safe_load(f)
  return data or {}


def _deep_merge(dst: dict, src: dict) -> dict:
  for k, v in src.items():
    if isinstance(v, dict) and isinstance(dst.get(k), dict):
      _deep_merge(dst[k], v)
    else:
      dst[k] = copy.deepcopy(v)
  return dst


def _set_path(tree: dict, path: list[str], value):
  node = tree
  for p in path[:-1]:
    nxt = node.get(p)
    if not isinstance(nxt, dict):
      nxt = {}
      node[p] = nxt
    node = nxt
  if isinstance(value, dict) and isinstance(node.get(path[-1]), dict):
    _deep_merge(node[path[-1]], value)
  else:
    node[path[-1]] = value


def _find_yaml(root: str, rel: str) -> str | None:
  for ext in (".yaml", ".yml"):
    p = os.path.join(root, rel + ext)
    if os.path.isfile(p):
      return p
  return None


class _Composer:
  def __init__(self, root: str, group_choices: dict[str, str]):
    self.root = root
    # group path relative to root ("model", "model/remat") -> chosen option
    self.choices = dict(group_choices)
    self.used_choices: set[str] = set()

  def load(self, rel_name: str, group_dir: str, package: list[str]) -> dict:
    """Compose file ``<root>/<group_dir>/<rel_name>.yaml`` placing content at ``package``."""
    rel = os.path.join(group_dir, rel_name) if group_dir else rel_name
    path = _find_yaml(self.root, rel)
    if path is None:
      avail = sorted(
        os.path.splitext(f)[0]
        for f in os.listdir(os.path.join(self.root, group_dir))
        if f.endswith((".yaml", ".yml"))
      ) if os.path.isdir(os.path.join(self.root, group_dir)) else []
      raise FileNotFoundError(
        f"config '{rel}' not found under {self.root}; available in '{group_dir or '.'}': {avail}"
      )
    raw = load_yaml(path)
    defaults = raw.pop("defaults", None)
    out: dict = {}
    if defaults is None:
      defaults = ["_self_"]
    if "_self_" not in defaults:
      # Hydra >= 1.1 composes the file itself last when _self_ is not listed.
      defaults = list(defaults) + ["_self_"]

    # "override group: option" entries in this file re-target groups that a
    # config named earlier in the list selects.
    for entry in defaults:
      if isinstance(entry, dict):
        for k, v in entry.items():
          if k.startswith("override "):
            grp = os.path.join(group_dir, k[len("override "):].strip()) if group_dir else k[len("override "):].strip()
            self.choices.setdefault(grp, v)

    for entry in defaults:
      if entry == "_self_":
        if package:
          _set_path(out, package, raw)
        else:
          _deep_merge(out, raw)
      elif isinstance(entry, str):
        # sibling config merged at the same package
        _deep_merge(out, self.load(entry, group_dir, package))
      elif isinstance(entry, dict):
        for k, v in entry.items():
          if k.startswith("override "):
            continue
          optional = k.startswith("optional ")
          grp_name = k[len("optional "):].strip() if optional else k
          grp_rel = os.path.join(group_dir, grp_name) if group_dir else grp_name
          option = self.choices.get(grp_rel, v)
          if grp_rel in self.choices:
            self.used_choices.add(grp_rel)
          if option is None:
            continue
          try:
            sub = self.load(str(option), grp_rel, package + grp_name.split("/"))
          except FileNotFoundError:
            if optional:
              continue
            raise
          _deep_merge(out, sub)
      else:
        raise ValueError(f"unsupported defaults entry {entry!r} in {path}")
    return out


def _parse_value(text: str):
  if text == "":
    return ""
  try:
    return yaml.safe_load(text)
  except yaml.YAMLError:
    return text


def parse_cli(argv: Iterable[str]) -> tuple[str | None, list[str]]:
  """Split ``--config-name X`` / ``--config-name=X`` from the override list."""
  config_name = None
  overrides: list[str] = []
  it = iter(argv)
  for a in it:
    if a in ("--config-name", "-cn"):
      config_name = next(it)
    elif a.startswith("--config-name="):
      config_name = a.split("=", 1)[1]
    else:
      overrides.append(a)
  return config_name, overrides


def compose(
  config_name: str = "default",
  overrides: Iterable[str] = (),
  config_root: str | None = None,
) -> Config:
  """Compose ``<config_root>/<config_name>.yaml`` with command-line overrides.

  Same surface as the reference's hydra entry (train.py:29): group selection
  (``model=mixtral-8x7b``, ``model/remat=llama-scan``), value overrides
  (``task.max_steps=5``), additions (``+a.b=1``) and deletions (``~a.b``).
  """
  root = config_root or CONFIG_ROOT
  overrides = list(overrides)
  group_choices: dict[str, str] = {}
  value_overrides: list[tuple[str, str, Any]] = []
  for ov in overrides:
    if ov.startswith("~"):
      value_overrides.append(("del", ov[1:].split("=")[0], None))
      continue
    if "=" not in ov:
      raise ValueError(f"override '{ov}' is not of the form key=value")
    key, val = ov.split("=", 1)
    mode = "set"
    if key.startswith("++"):
      key, mode = key[2:], "force"
    elif key.startswith("+"):
      key, mode = key[1:], "add"
    is_group = (
      mode == "set"
      and os.path.isdir(os.path.join(root, key))
      and "." not in key
      and _find_yaml(root, os.path.join(key, val)) is not None
    )
    if is_group:
      group_choices[key] = val
    else:
      value_overrides.append((mode, key, _parse_value(val)))

  comp = _Composer(root, group_choices)
  tree = comp.load(config_name, "", [])
  unused = set(group_choices) - comp.used_choices
  # A group chosen on the command line that no defaults list mentions is
  # appended (hydra would need "+group=opt"; being lenient here is harmless).
  for grp in sorted(unused):
    sub = comp.load(group_choices[grp], grp, grp.split("/"))
    _deep_merge(tree, sub)

  for mode, key, val in value_overrides:
    path = key.split(".")
    if mode == "del":
      node = tree
      for p in path[:-1]:
        node = node.get(p, {})
      node.pop(path[-1], None)
      continue
    if mode == "set":
      node = tree
      ok = True
      for p in path:
        if isinstance(node, dict) and p in node:
          node = node[p]
        else:
          ok = False
          break
      if not ok:
        raise KeyError(
          f"override '{key}' does not name an existing config key; use '+{key}=...' to add it"
        )
    _set_path(tree, path, val)
  return Config(tree)
