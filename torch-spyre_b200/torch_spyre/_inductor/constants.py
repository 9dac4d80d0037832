DEVICE_NAME = "spyre"
