package neureka.devices.cuda;

import neureka.Data;
import neureka.Tensor;
import neureka.backend.api.ExecutionCall;
import neureka.backend.api.Operation;
import neureka.common.composition.Component.OwnerChangeRequest;
import neureka.devices.AbstractDevice;
import neureka.devices.Device;
import neureka.dtype.DataType;
import neureka.math.Function;
import neureka.ndim.config.NDConfiguration;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;
import java.lang.foreign.ValueLayout;
import java.util.Collection;
import java.util.Collections;
import java.util.Set;
import java.util.WeakHashMap;

/**
 *  neureka.devices.Device for one B200, replacing OpenCLDevice's memory handling (OpenCLDevice.java:316-334 restore,
 *  :355-405 store, :497-524 free, :553-594 allocate, :616-632 overwrite, :676-690 read). F64 is first class: there is no
 *  down-cast on store. The executable twin of this class, used by the parity tests, is neureka_b200/device.py.
 *  COMPILE-UNVERIFIED (no JDK where this repository is built).
 */
public final class CudaDevice extends AbstractDevice<Number>
{
    final MemorySegment ctx;   // nk_ctx*
    private final int _ordinal;
    private final Set<Tensor<Number>> _tensors = Collections.newSetFromMap(new WeakHashMap<>());

    public CudaDevice( int ordinal ) {
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment out = a.allocate(ValueLayout.ADDRESS);
            NeurekaCuda.check((int) NeurekaCuda.DEVICE_OPEN.invokeExact(ordinal, out), MemorySegment.NULL);
            ctx = out.get(ValueLayout.ADDRESS, 0);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        _ordinal = ordinal;
    }

    /** Number of CUDA devices the library sees (nk_device_count). */
    public static int count() {
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment out = a.allocate(ValueLayout.JAVA_INT);
            NeurekaCuda.check((int) NeurekaCuda.DEVICE_COUNT.invokeExact(out), MemorySegment.NULL);
            return out.get(ValueLayout.JAVA_INT, 0);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
    }

    public int ordinal() { return _ordinal; }

    static int typeOf( Class<?> c ) {
        if ( c == Float.class   ) return NeurekaCuda.F32;
        if ( c == Double.class  ) return NeurekaCuda.F64;
        if ( c == Byte.class    ) return NeurekaCuda.I8;
        if ( c == Short.class   ) return NeurekaCuda.I16;
        if ( c == Integer.class ) return NeurekaCuda.I32;
        if ( c == Long.class    ) return NeurekaCuda.I64;
        throw new IllegalArgumentException("Data type '" + c + "' cannot be stored on a CudaDevice");
    }

    void _free( MemorySegment buf ) {
        try { NeurekaCuda.check((int) NeurekaCuda.FREE.invokeExact(ctx, buf), ctx); }
        catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
    }

    private <T extends Number> CudaData<T> _alloc( DataType<T> type, long size ) {
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment out = a.allocate(ValueLayout.ADDRESS);
            NeurekaCuda.check((int) NeurekaCuda.ALLOC.invokeExact(ctx, typeOf(type.getItemTypeClass()), size, out), ctx);
            return new CudaData<>(this, out.get(ValueLayout.ADDRESS, 0), size, type);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
    }

    /** The nk_buf of a tensor stored here (KernelCaller.passAllOf reads the cl_mem the same way, KernelCaller.java:41-46). */
    MemorySegment bufOf( Tensor<?> t ) { return ((CudaData<?>) t.mut().getData()).buf; }

    // ---- Device / Storage -----------------------------------------------------------------------------------------

    @Override public <T extends Number> Data<T> allocate( DataType<T> type, NDConfiguration ndc ) { return _alloc(type, ndc.size()); }

    @Override public <T extends Number> Data<T> allocateFromOne( DataType<T> type, NDConfiguration ndc, T initial ) {
        CudaData<T> d = _alloc(type, ndc.size());
        try { NeurekaCuda.check((int) NeurekaCuda.FILL.invokeExact(ctx, d.buf, initial.doubleValue(), 0L, d.size), ctx); }
        catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return d;
    }

    @Override public <T extends Number> Data<T> allocateFromAll( DataType<T> type, NDConfiguration ndc, Object jvmData ) {
        MemorySegment heap = heapSegment(jvmData);
        long n = heap.byteSize() / bytesOf(type.getItemTypeClass());
        CudaData<T> d = _alloc(type, Math.max(n, ndc.size()));
        try ( Arena a = Arena.ofConfined() ) {
            // FFM cannot pass heap segments to a downcall that keeps no critical section: stage through native memory
            MemorySegment staged = a.allocate(heap.byteSize(), 64).copyFrom(heap);
            NeurekaCuda.check((int) NeurekaCuda.WRITE.invokeExact(ctx, d.buf, staged, 0L, 0L, n), ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return d;
    }

    @Override public boolean update( OwnerChangeRequest<Tensor<Number>> changeRequest ) {
        // store(tensor) arrives here (AbstractDevice.java:87-108): upload like OpenCLDevice._add (:355-405); slices share
        // their root's CudaData; a virtual tensor uploads one element; an attached gradient migrates too.
        super.update(changeRequest);
        Tensor<Number> t = changeRequest.getNewOwner();
        if ( t != null && !_tensors.contains(t) ) {
            Object jvm = t.mut().getData().getOrNull();
            Data<Number> data = allocateFromAll((DataType<Number>) t.getDataType(), t.getNDConf(), jvm);
            t.mut().setData(data);
            _tensors.add(t);
            if ( t.hasGradient() ) this.store(t.gradient().get());
        }
        return changeRequest.executeChange();
    }

    @Override public Device<Number> restore( Tensor<Number> t ) {
        if ( !has(t) ) throw new IllegalStateException("The given tensor is not stored on this device");
        Object all = _readAll(t, true);
        free(t);
        t.mut().setItems(all);
        return this;
    }

    @Override public <T extends Number> Device<Number> free( Tensor<T> t ) {
        _tensors.remove(t);
        t.mut().setData(null);   // dropping the last usage runs CudaData's cleanup -> nk_free
        return this;
    }

    @Override public <T extends Number> boolean has( Tensor<T> t ) { return _tensors.contains(t); }
    @Override public boolean contains( Tensor<Number> t ) { return has(t); }
    @Override public int numberOfStored() { return _tensors.size(); }
    @Override public boolean isEmpty() { return _tensors.isEmpty(); }
    @Override public Collection<Tensor<Number>> getTensors() { return _tensors; }
    /**
     *  Device.optimizedOperationOf (Device.java:216-241; model: CLFunctionCompiler.java:47-196): the Function tree is
     *  turned into the expression language of nk_fused_compile and wrapped into an Operation whose execution is a
     *  single nk_fused_run. Operands may broadcast, which the OpenCL compiler of the reference does not support.
     */
    @Override public Operation optimizedOperationOf( Function function, String name ) {
        final String expr = CudaKernels.fusedExpressionOf( function );
        final int arity = function.numberOfArgs();
        return Operation.builder()
                .identifier( name ).operator( name ).arity( arity )
                .isOperator( false ).isIndexer( false ).isDifferentiable( false ).isInline( false )
                .stringifier( children -> name + "(" + String.join(", ", children) + ")" )
                .build()
                .setAlgorithm(
                    neureka.backend.api.template.algorithms.FunDeviceAlgorithm.withName("generic_algorithm_for_" + name)
                        .setIsSuitableFor( call -> neureka.backend.api.fun.SuitabilityPredicate.GOOD )
                        .setAutogradModeFor( call -> neureka.backend.api.AutoDiffMode.NOT_SUPPORTED )
                        .setExecution( (outerCaller, outerCall) -> neureka.backend.api.Result.of(
                            CudaKernels.runFused( this, expr, arity, outerCall ) ) )
                        .buildFunAlgorithm()
                );
    }
    @Override public void dispose() {
        _tensors.clear();
        try { NeurekaCuda.check((int) NeurekaCuda.DEVICE_CLOSE.invokeExact(ctx), MemorySegment.NULL); }
        catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
    }

    // ---- AbstractDevice hooks ---------------------------------------------------------------------------------------

    @Override protected boolean _approveExecutionOf( Tensor<?>[] tensors, int d, Operation type ) { return true; }
    @Override protected <T extends Number> void _swap( Tensor<T> former, Tensor<T> replacement ) { _tensors.remove(former); _tensors.add((Tensor<Number>) replacement); }
    @Override protected <T extends Number> int _sizeOccupiedBy( Tensor<T> t ) { return (int) ((CudaData<?>) t.mut().getData()).size; }
    @Override protected <T extends Number> Object _readAll( Tensor<T> t, boolean clone ) { return _readArray(t, arrayTypeOf(t), 0, _sizeOccupiedBy(t)); }
    @Override protected <T extends Number> T _readItem( Tensor<T> t, int index ) { return (T) java.lang.reflect.Array.get(_readArray(t, arrayTypeOf(t), index, 1), 0); }

    @Override protected <T extends Number, A> A _readArray( Tensor<T> t, Class<A> arrayType, int start, int size ) {
        Object array = java.lang.reflect.Array.newInstance(arrayType.getComponentType(), size);
        MemorySegment heap = heapSegment(array);
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment staged = a.allocate(heap.byteSize(), 64);
            NeurekaCuda.check((int) NeurekaCuda.READ.invokeExact(ctx, bufOf(t), staged, (long) start, (long) size), ctx);   // blocking
            heap.copyFrom(staged);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable th ) { throw new IllegalStateException(th); }
        return (A) array;
    }

    @Override protected <T extends Number> void _writeItem( Tensor<T> t, T item, int start, int size ) {
        try { NeurekaCuda.check((int) NeurekaCuda.FILL.invokeExact(ctx, bufOf(t), item.doubleValue(), (long) start, (long) size), ctx); }
        catch ( RuntimeException e ) { throw e; } catch ( Throwable th ) { throw new IllegalStateException(th); }
    }

    @Override protected <T extends Number> void _writeArray( Tensor<T> t, Object array, int offset, int start, int size ) {
        MemorySegment heap = heapSegment(array);
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment staged = a.allocate(heap.byteSize(), 64).copyFrom(heap);
            NeurekaCuda.check((int) NeurekaCuda.WRITE.invokeExact(ctx, bufOf(t), staged, (long) offset, (long) start, (long) size), ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable th ) { throw new IllegalStateException(th); }
    }

    @Override protected Data<Number> _actualize( Tensor<?> t ) {
        // one element -> size copies of it (OpenCLDevice.java:574-585)
        Number v = _readItem((Tensor<Number>) t, 0);
        return allocateFromOne((DataType<Number>) t.getDataType(), t.getNDConf(), v);
    }

    @Override protected Data<Number> _virtualize( Tensor<?> t ) {
        Number v = _readItem((Tensor<Number>) t, 0);
        CudaData<Number> d = _alloc((DataType<Number>) t.getDataType(), 1);
        _writeItemInto(d, v);
        return d;
    }

    private void _writeItemInto( CudaData<?> d, Number v ) {
        try { NeurekaCuda.check((int) NeurekaCuda.FILL.invokeExact(ctx, d.buf, v.doubleValue(), 0L, 1L), ctx); }
        catch ( RuntimeException e ) { throw e; } catch ( Throwable th ) { throw new IllegalStateException(th); }
    }

    @Override protected DataType<?> _dataTypeOf( Object rawData ) { return DataType.of(rawData.getClass().getComponentType()); }

    private static Class<?> arrayTypeOf( Tensor<?> t ) {
        Class<?> c = t.getItemType();
        if ( c == Float.class ) return float[].class;
        if ( c == Double.class ) return double[].class;
        if ( c == Integer.class ) return int[].class;
        if ( c == Long.class ) return long[].class;
        if ( c == Short.class ) return short[].class;
        return byte[].class;
    }

    private static long bytesOf( Class<?> c ) { return ( c == Double.class || c == Long.class ) ? 8 : ( c == Float.class || c == Integer.class ) ? 4 : ( c == Short.class ) ? 2 : 1; }

    private static MemorySegment heapSegment( Object array ) {
        if ( array instanceof float[]  a ) return MemorySegment.ofArray(a);
        if ( array instanceof double[] a ) return MemorySegment.ofArray(a);
        if ( array instanceof int[]    a ) return MemorySegment.ofArray(a);
        if ( array instanceof long[]   a ) return MemorySegment.ofArray(a);
        if ( array instanceof short[]  a ) return MemorySegment.ofArray(a);
        if ( array instanceof byte[]   a ) return MemorySegment.ofArray(a);
        throw new IllegalArgumentException("Unsupported array type " + array.getClass());
    }

    @Override public String toString() { return "CudaDevice[" + _ordinal + "]"; }
}
