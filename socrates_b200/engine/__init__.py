"""Step function, scheduler, Python entry point and trace replay."""
