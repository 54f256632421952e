"""``coda.core.elementwise`` of the drop-in layout: the element-wise operators under the reference's names."""
