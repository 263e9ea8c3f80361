"""Engine assembly: checkpoint detection, runtime construction, the adapter the backend drives."""
