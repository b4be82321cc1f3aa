from . import meta, qlayer  # noqa: F401
