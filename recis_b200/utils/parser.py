"""Dataclass-driven argument parser (role of ``recis/utils/parser.py:4-86``, which wraps ``simple_parsing``).
``add_arguments(DataclassType, dest="name")`` registers every field as ``--name.field`` (and ``--field`` when unambiguous);
``parse_args()`` returns a namespace whose ``name`` attribute is an instance of the dataclass."""
from __future__ import annotations

import argparse
import dataclasses
import typing


def _convert(tp, text):
    origin = typing.get_origin(tp)
    if origin is typing.Union:
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        if text in ("None", "none", ""):
            return None
        return _convert(args[0], text)
    if tp is bool:
        return text.lower() in ("1", "true", "yes", "y")
    if origin in (list, typing.List) or tp is list:
        inner = (typing.get_args(tp) or (str,))[0]
        return [_convert(inner, t) for t in text.split(",") if t != ""]
    if tp in (int, float, str):
        return tp(text)
    return text


class ArgumentParser(argparse.ArgumentParser):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._groups = []
        self._short = {}

    def add_arguments(self, dataclass_type, dest: str, default=None):
        assert dataclasses.is_dataclass(dataclass_type)
        self._groups.append((dataclass_type, dest, default))
        hints = typing.get_type_hints(dataclass_type)
        for f in dataclasses.fields(dataclass_type):
            names = [f"--{dest}.{f.name}"]
            if f.name not in self._short:
                self._short[f.name] = dest
                names.append(f"--{f.name}")
            self.add_argument(*names, dest=f"{dest}.{f.name}", type=str, default=None, help=f"{hints.get(f.name, str)}")

    def parse_args(self, args=None, namespace=None):
        ns = super().parse_args(args, namespace)
        for dc, dest, default in self._groups:
            hints = typing.get_type_hints(dc)
            values = {}
            for f in dataclasses.fields(dc):
                raw = getattr(ns, f"{dest}.{f.name}")
                if raw is not None:
                    values[f.name] = _convert(hints.get(f.name, str), raw)
                delattr(ns, f"{dest}.{f.name}")
            base = default if default is not None else dc()
            setattr(ns, dest, dataclasses.replace(base, **values))
        return ns
