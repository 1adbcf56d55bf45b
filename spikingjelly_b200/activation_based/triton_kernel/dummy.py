"""Placeholder object for an optional dependency that is absent: every attribute, call and item of it is another
placeholder, and it is false in a boolean test (``triton_kernel/dummy.py`` of the reference, where it stands in for the
``triton`` module)."""

__all__ = ["DummyImport"]


class DummyImport:
    def __getattr__(self, name):
        return DummyImport()

    def __call__(self, *args, **kwargs):
        return DummyImport()

    def __getitem__(self, item):
        return DummyImport()

    def __bool__(self):
        return False

    def __repr__(self):
        return "<DummyImport>"
