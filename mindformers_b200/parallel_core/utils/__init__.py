"""``parallel_core/utils`` of the reference: module specs and initialisers."""
