"""Record format, calibration tables and the device-backed record codec."""
