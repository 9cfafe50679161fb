"""Side scripts that are not part of the training framework proper."""
