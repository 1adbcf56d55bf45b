import threading
_tls = threading.local()


def in_gc_1st_forward() -> bool:
    return getattr(_tls, "flag", False)
