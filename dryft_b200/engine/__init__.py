"""The engine: model assembly, the step function, the generation loop and the Python entry point."""
