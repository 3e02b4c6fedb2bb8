package neureka.devices.cuda;

import neureka.devices.AbstractDeviceData;
import neureka.dtype.DataType;

import java.lang.foreign.MemorySegment;

/**
 *  Device memory of one tensor family (a root tensor and all its slices): an nk_buf handle, reference-counted by
 *  tensor usage exactly like the OpenCL counterpart (OpenCLDevice.java:954-966); the cleanup runs nk_free, possibly
 *  on the "Neureka-Cleaner" thread -- nk_free sets the CUDA device itself, so any thread may call it.
 *  COMPILE-UNVERIFIED.
 */
final class CudaData<T> extends AbstractDeviceData<T>
{
    final MemorySegment buf;   // nk_buf*
    final long size;           // elements

    CudaData( CudaDevice owner, MemorySegment buf, long size, DataType<T> type ) {
        super( owner, buf, type, () -> owner._free( buf ) );
        this.buf = buf;
        this.size = size;
    }
}
