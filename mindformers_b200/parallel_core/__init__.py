"""The reference's ``mindformers/parallel_core`` import paths. The implementation is ``mindformers_b200/parallel`` (one set of layers serves training and inference)."""
