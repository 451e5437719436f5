"""Build output folder of the sm_100a kernel library (``libtitan_b200.so``)."""
