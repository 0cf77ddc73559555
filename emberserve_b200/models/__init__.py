"""Built-in architectures (Qwen2 dense, Damolorn, Dedizen).  Importing this package registers them."""

from emberserve_b200.models import damolorn, dedizen, qwen2  # noqa: F401
