"""Dataclass-driven argument parser with the calling convention of Hugging Face's
``HfArgumentParser`` (which the reference vendors, hf_argparser.py:124-473): one ``--flag`` per
dataclass field, booleans written as ``--flag True|False`` (or bare ``--flag``), ``Optional[T]``
fields, ``Path`` fields, and JSON / YAML / dict loaders. Written from scratch against that
interface; only the features the entry points use are implemented.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys
import types
import typing
from enum import Enum
from pathlib import Path
from typing import Any, Iterable, List, Optional, Tuple, Union

_TRUE = {"yes", "true", "t", "y", "1"}
_FALSE = {"no", "false", "f", "n", "0"}


def string_to_bool(v: Union[str, bool]) -> bool:
    if isinstance(v, bool):
        return v
    s = str(v).strip().lower()
    if s in _TRUE:
        return True
    if s in _FALSE:
        return False
    raise argparse.ArgumentTypeError(
        f"Truthy value expected: got {v!r} but expected one of yes/no, true/false, t/f, y/n, 1/0")


def _strip_optional(tp):
    """Optional[T] -> (T, True); T -> (T, False)."""
    origin = typing.get_origin(tp)
    if origin is Union or origin is getattr(types, "UnionType", None):
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        if len(args) == 1:
            return args[0], True
        if str in args:  # e.g. Union[int, str]: parse as str
            return str, True
        return args[0], True
    return tp, False


class HfArgumentParser(argparse.ArgumentParser):
    def __init__(self, dataclass_types, **kwargs):
        kwargs.setdefault("formatter_class", argparse.ArgumentDefaultsHelpFormatter)
        super().__init__(**kwargs)
        if dataclasses.is_dataclass(dataclass_types):
            dataclass_types = [dataclass_types]
        self.dataclass_types = list(dataclass_types)
        for dt in self.dataclass_types:
            self._add_dataclass_arguments(dt)

    # ------------------------------------------------------------------ declaration
    def _add_dataclass_arguments(self, dtype) -> None:
        try:
            hints = typing.get_type_hints(dtype)
        except Exception:
            hints = {f.name: f.type for f in dataclasses.fields(dtype)}
        for f in dataclasses.fields(dtype):
            if not f.init:
                continue
            self._add_field(f, hints.get(f.name, f.type))

    def _add_field(self, f: dataclasses.Field, ftype) -> None:
        name = f"--{f.name}"
        kw: dict = {"help": f.metadata.get("help")}
        aliases = f.metadata.get("aliases", [])
        if isinstance(aliases, str):
            aliases = [aliases]
        base, optional = _strip_optional(ftype)
        has_default = f.default is not dataclasses.MISSING
        has_factory = f.default_factory is not dataclasses.MISSING
        origin = typing.get_origin(base)
        if isinstance(base, type) and issubclass(base, Enum):
            kw["choices"] = [e.value for e in base]
            kw["type"] = type(kw["choices"][0])
        elif origin is typing.Literal:
            kw["choices"] = list(typing.get_args(base))
            kw["type"] = type(kw["choices"][0])
        elif base is bool:
            kw["type"] = string_to_bool
            kw["nargs"] = "?"
            kw["const"] = True
            kw["metavar"] = "BOOL"
        elif origin in (list, List):
            kw["nargs"] = "+"
            kw["type"] = typing.get_args(base)[0]
        else:
            kw["type"] = base
        if has_default:
            kw["default"] = f.default
        elif has_factory:
            kw["default"] = f.default_factory()
        elif optional:
            kw["default"] = None
        else:
            kw["required"] = True
        self.add_argument(name, *aliases, **kw)
        if base is bool and has_default and f.default is True:
            # a default-True flag also gets a --no_<name> switch
            self.add_argument(f"--no_{f.name}", action="store_false", dest=f.name,
                              help=argparse.SUPPRESS)

    # ------------------------------------------------------------------ parsing
    def parse_args_into_dataclasses(self, args: Optional[Iterable[str]] = None,
                                    return_remaining_strings: bool = False,
                                    look_for_args_file: bool = True,
                                    args_filename: Optional[str] = None,
                                    args_file_flag: Optional[str] = None) -> Tuple[Any, ...]:
        argv = list(sys.argv[1:] if args is None else args)
        file_args: List[str] = []
        if args_filename:
            file_args += Path(args_filename).read_text().split()
        elif look_for_args_file and len(sys.argv) and args is None:
            cand = Path(sys.argv[0]).with_suffix(".args")
            if cand.exists():
                file_args += cand.read_text().split()
        if args_file_flag and args_file_flag in argv:
            i = argv.index(args_file_flag)
            file_args += Path(argv[i + 1]).read_text().split()
            del argv[i: i + 2]
        namespace, remaining = self.parse_known_args(file_args + argv)
        outputs = self._namespace_to_dataclasses(vars(namespace))
        if return_remaining_strings:
            return (*outputs, remaining)
        if remaining:
            raise ValueError(f"Some specified arguments are not used by the parser: {remaining}")
        return tuple(outputs)

    def _namespace_to_dataclasses(self, values: dict) -> list:
        outs = []
        for dt in self.dataclass_types:
            keys = {f.name for f in dataclasses.fields(dt) if f.init}
            outs.append(dt(**{k: v for k, v in values.items() if k in keys}))
        return outs

    def parse_dict(self, args: dict, allow_extra_keys: bool = False) -> Tuple[Any, ...]:
        used = set()
        outs = []
        for dt in self.dataclass_types:
            keys = {f.name for f in dataclasses.fields(dt) if f.init}
            outs.append(dt(**{k: v for k, v in args.items() if k in keys}))
            used |= keys & set(args)
        extra = set(args) - used
        if extra and not allow_extra_keys:
            raise ValueError(f"Some keys are not used by the HfArgumentParser: {sorted(extra)}")
        return tuple(outs)

    def parse_json_file(self, json_file: str, allow_extra_keys: bool = False):
        with open(Path(json_file), encoding="utf-8") as fh:
            return self.parse_dict(json.load(fh), allow_extra_keys=allow_extra_keys)

    def parse_yaml_file(self, yaml_file: str, allow_extra_keys: bool = False):
        import yaml
        return self.parse_dict(yaml.safe_load(Path(yaml_file).read_text()),
                               allow_extra_keys=allow_extra_keys)
