from .composer import CONFIG_ROOT, Config, compose, load_yaml, parse_cli, to_container

__all__ = ["CONFIG_ROOT", "Config", "compose", "load_yaml", "parse_cli", "to_container"]
