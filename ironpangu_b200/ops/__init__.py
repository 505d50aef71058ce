"""ops sub-package."""
