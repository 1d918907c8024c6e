"""Built-in architectures (Qwen2 dense, Damolorn, Dedizen, Vonulix, Lesosun).  Importing this package registers them."""

from emberserve_b200.models import damolorn, dedizen, lesosun, qwen2, vonulix  # noqa: F401
