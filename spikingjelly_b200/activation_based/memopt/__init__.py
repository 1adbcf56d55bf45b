from .checkpointing import in_gc_1st_forward  # noqa: F401
