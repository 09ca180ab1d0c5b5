"""``DataRecord``: the small key → value store that the modal builders fill while a query is pre-processed (reference
``models/multi_modal/utils.py:21``)."""
from __future__ import annotations


class DataRecord:
    def __init__(self):
        self.data = {}

    def put(self, key, value, append: bool = False):
        """Set ``key``; with ``append`` the values of a key collect in a list."""
        if append:
            self.data.setdefault(key, []).append(value)
        else:
            self.data[key] = value

    def put_from_dict(self, dict_):
        for key, value in dict_.items():
            self.put(key, value)

    def get(self, key):
        return self.data.get(key)

    def has_key(self, key) -> bool:
        return key in self.data

    def output(self, keys, format_: str = "dict"):
        if format_ == "tuple":
            return tuple(self.get(k) for k in keys)
        if format_ == "dict":
            return {k: self.get(k) for k in keys}
        raise ValueError(f"format={format_} is not supported.")

    def clear(self):
        self.data = {}
