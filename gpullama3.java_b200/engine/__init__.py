"""The engine: the model assembled from parts, the step function, generation, trace replay."""
