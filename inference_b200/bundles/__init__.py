"""Runtime bundles: `runtime_b200.catalog()` and `runtime_cpu.catalog()` return validated catalogs."""
from . import runtime_b200, runtime_cpu  # noqa: F401
from .catalog import AudioSection, RuntimeCatalog, RuntimeCatalogError, RuntimeCatalogSnapshot  # noqa: F401
