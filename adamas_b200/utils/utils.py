"""Cache-page layout names shared by the host runtime and the operators."""
from __future__ import annotations


class _LayoutNamespace(type):
    """Class-level helpers for TensorLayout: the layout codes are plain ints (they travel through the C ABI
    as such), this only adds lookups in both directions and iteration over the known layouts."""

    def __iter__(cls):
        return iter(sorted(cls.FORMAT2STR))

    def __contains__(cls, code) -> bool:
        return code in cls.FORMAT2STR


class TensorLayout(metaclass=_LayoutNamespace):
    """Order of the last three dimensions of a cache page: tokens-heads-dim or heads-tokens-dim.  The
    attribute names and values are the ones the reference's operators take (adamas/utils/utils.py:1-5);
    this library implements tokens-heads-dim only and rejects the other with an error."""

    FORMAT2STR = dict(enumerate(("NHD", "HND")))
    NHD, HND = sorted(FORMAT2STR)

    @classmethod
    def name_of(cls, code: int) -> str:
        return cls.FORMAT2STR[int(code)]

    @classmethod
    def parse(cls, name: str) -> int:
        for code, text in cls.FORMAT2STR.items():
            if text == name:
                return code
        raise KeyError(f"unknown cache layout {name!r}")
