"""search subpackage."""
