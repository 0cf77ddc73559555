"""Built-in architectures (Qwen2 dense, Damolorn).  Importing this package registers them."""

from emberserve_b200.models import damolorn, qwen2  # noqa: F401
