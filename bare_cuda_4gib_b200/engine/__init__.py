"""The engine: generic model, step function, scheduler and entry points."""
