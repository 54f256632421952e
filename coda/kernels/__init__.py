"""Operator packages of the drop-in layout (see ``coda/__init__.py``)."""
