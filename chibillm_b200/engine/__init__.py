"""Engine: batches, the model, the step function, the scheduler and the loop."""
