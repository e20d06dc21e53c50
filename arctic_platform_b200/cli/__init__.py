"""Small command-line helpers shipped with the package (``python -m arctic_platform_b200.cli.<name>``)."""
