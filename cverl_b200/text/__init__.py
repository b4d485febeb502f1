"""text subpackage."""
