"""Helper modules of the drop-in layout (see ``coda/__init__.py``)."""
