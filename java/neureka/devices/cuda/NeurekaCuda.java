package neureka.devices.cuda;

import java.lang.foreign.*;
import java.lang.invoke.MethodHandle;

import static java.lang.foreign.ValueLayout.*;

/**
 *  Panama FFM (JDK 22+) binding of the C ABI in include/neureka_cuda.h. One static MethodHandle per entry point;
 *  no JNI, no generated code. COMPILE-UNVERIFIED: the image this repository is built in has no JDK.
 *  Status codes are turned into the exception types Neureka's implementations throw:
 *  NK_ERR_BAD_ARG / NK_ERR_UNSUPPORTED / NK_ERR_BOUNDS -> IllegalArgumentException, everything else -> IllegalStateException.
 */
public final class NeurekaCuda
{
    public static final int F32 = 0, F64 = 1, I8 = 2, I16 = 3, I32 = 4, I64 = 5;
    public static final int OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_DIV = 3, OP_MOD = 4, OP_POW = 5, OP_IDY = 6;

    private static final Linker LINKER = Linker.nativeLinker();
    private static final SymbolLookup LIB = SymbolLookup.libraryLookup(
            System.getProperty("neureka.cuda.library", "libneureka_cuda.so"), Arena.global());

    private static MethodHandle h( String name, FunctionDescriptor d ) {
        return LINKER.downcallHandle( LIB.find(name).orElseThrow(() -> new UnsatisfiedLinkError(name)), d );
    }

    static final MethodHandle DEVICE_COUNT = h("nk_device_count", FunctionDescriptor.of(JAVA_INT, ADDRESS));
    static final MethodHandle DEVICE_OPEN  = h("nk_device_open",  FunctionDescriptor.of(JAVA_INT, JAVA_INT, ADDRESS));
    static final MethodHandle DEVICE_CLOSE = h("nk_device_close", FunctionDescriptor.of(JAVA_INT, ADDRESS));
    static final MethodHandle SYNC         = h("nk_sync",         FunctionDescriptor.of(JAVA_INT, ADDRESS));
    static final MethodHandle LAST_ERROR   = h("nk_last_error",   FunctionDescriptor.of(ADDRESS, ADDRESS));
    static final MethodHandle ALLOC        = h("nk_alloc",        FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_LONG, ADDRESS));
    static final MethodHandle FREE         = h("nk_free",         FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS));
    static final MethodHandle FILL         = h("nk_fill",         FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_DOUBLE, JAVA_LONG, JAVA_LONG));
    static final MethodHandle WRITE        = h("nk_write",        FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_LONG, JAVA_LONG, JAVA_LONG));
    static final MethodHandle READ         = h("nk_read",         FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_LONG, JAVA_LONG));
    static final MethodHandle COPY         = h("nk_copy",         FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_LONG, ADDRESS, JAVA_LONG, JAVA_LONG));
    static final MethodHandle CONV         = h("nk_conv",         FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT));
    static final MethodHandle BROADCAST    = h("nk_broadcast",    FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT));
    static final MethodHandle BINARY       = h("nk_binary",       FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT));
    static final MethodHandle UNARY        = h("nk_unary",        FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT));
    static final MethodHandle SCALAR_BIN   = h("nk_scalar_binary",FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_DOUBLE, JAVA_INT));
    static final MethodHandle FILL_FUN     = h("nk_fill_fun",     FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, JAVA_DOUBLE, JAVA_INT));
    static final MethodHandle SUM          = h("nk_sum",          FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_LONG));

    // Min / Max: the flat index of the extreme element, written as one int into a device buffer (CLReduce's contract)
    static final MethodHandle ARG_REDUCE   = h("nk_arg_reduce",   FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_LONG));

    static final MethodHandle FUSED_COMPILE = h("nk_fused_compile", FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS));
    static final MethodHandle FUSED_RUN     = h("nk_fused_run",     FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS));
    static final MethodHandle FUSED_FREE    = h("nk_fused_free",    FunctionDescriptor.of(JAVA_INT, ADDRESS));
    // backward of a fused expression w.r.t. one input, reduction over that input's broadcast dims included
    static final MethodHandle FUSED_COMPILE_GRAD = h("nk_fused_compile_grad", FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS));
    static final MethodHandle FUSED_RUN_GRAD     = h("nk_fused_run_grad",     FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS));

    // memory a second process may open (nk_ipc_export); everything else comes from the stream-ordered pool behind nk_alloc
    static final MethodHandle ALLOC_SHARED  = h("nk_alloc_shared",  FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_LONG, ADDRESS));

    // several GPUs in this JVM: one context per member, peer access enabled once, halo-split convolution across the members
    static final MethodHandle GROUP_OPEN    = h("nk_group_open",    FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, ADDRESS));
    static final MethodHandle GROUP_SIZE    = h("nk_group_size",    FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS));
    static final MethodHandle GROUP_CTX     = h("nk_group_ctx",     FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, ADDRESS));
    static final MethodHandle GROUP_CLOSE   = h("nk_group_close",   FunctionDescriptor.of(JAVA_INT, ADDRESS));
    static final MethodHandle GROUP_PLAN    = h("nk_group_plan_slabs", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS, ADDRESS, ADDRESS));
    static final MethodHandle CONV_SHARDED  = h("nk_conv_sharded",  FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS));

    private NeurekaCuda() {}

    /** Converts a non-zero status into the exception the reference's implementations would throw. */
    static void check( int status, MemorySegment ctx ) {
        if ( status == 0 ) return;
        String msg;
        try { msg = ((MemorySegment) LAST_ERROR.invokeExact(ctx)).reinterpret(1024).getString(0); }
        catch ( Throwable t ) { msg = "status " + status; }
        if ( status == 1 || status == 2 || status == 6 ) throw new IllegalArgumentException(msg);
        throw new IllegalStateException(msg);
    }

    /** NDConfiguration.asInlineArray() copied into native memory for the duration of one call. */
    static MemorySegment cfg( Arena arena, int[] inline ) { return arena.allocateFrom(JAVA_INT, inline); }
}
