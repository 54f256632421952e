"""``coda.core.ops`` of the drop-in layout: only ``rope_utils`` is provided."""
