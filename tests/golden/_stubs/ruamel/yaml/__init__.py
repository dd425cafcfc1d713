"""Minimal stand-in for ruamel.yaml so the reference imports on this image (used only by make_golden.py)."""
import yaml as _y


class YAML:
    def __init__(self, *a, **k):
        self.default_flow_style = None

    def load(self, s):
        return _y.safe_load(s)

    def dump(self, obj, stream):
        stream.write(_y.safe_dump(obj).encode())
