"""runtime sub-package."""
