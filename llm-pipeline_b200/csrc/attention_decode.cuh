// Constants shared by the decode attention kernels and their merge kernel.
#pragma once

// Keys per range. Ranges are aligned to key 0, so a key's range depends on its index alone; every
// range of a row leaves one partial result (running max, running sum, vector) in scratch memory.
#define DEC_SPLIT 128
