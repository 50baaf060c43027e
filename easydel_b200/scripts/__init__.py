"""Command-line utilities (``python -m easydel_b200.scripts.<name>``)."""
