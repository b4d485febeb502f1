"""trainer subpackage."""
