"""Host utilities: NVLink check, failure detection, clock sampling, timing."""
