"""`import autort` for scripts written against the reference's AutoRT package: the same
export / ops / device surface, served by the antares_b200 kernel library."""
from antares_b200.autort_api import device, export, ops  # noqa: F401
