/* Stand-in for the JDK's <jni.h>, only for compiling the reference's cu32 libraries as a test
 * oracle on a machine without a JDK (TEST INFRASTRUCTURE, not product code).  It forwards to the
 * specification-conformant subset the product's own shim uses and adds the few names the
 * reference's JNITool.cuh touches (GetMethodID, NewObject, NewStringUTF, Throw). */
#ifndef ORACLE_JNI_STUB_H
#define ORACLE_JNI_STUB_H
#include <stdarg.h>
#include <stdint.h>

typedef int32_t jint;
typedef int64_t jlong;
typedef uint8_t jboolean;
typedef float jfloat;
typedef double jdouble;
typedef int8_t jbyte;
typedef uint16_t jchar;
typedef int16_t jshort;
typedef jint jsize;
struct _jobject;
typedef struct _jobject* jobject;
typedef jobject jclass;
typedef jobject jarray;
typedef jarray jlongArray;
typedef jobject jstring;
typedef jobject jthrowable;
struct _jmethodID;
typedef struct _jmethodID* jmethodID;
#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL
#define JNI_FALSE 0
#define JNI_TRUE 1

struct JNINativeInterface_ {
    void* slot[235];
};

struct JNIEnv_ {
    const struct JNINativeInterface_* functions;
    jclass FindClass(const char* name)
    {
        typedef jclass (*fn)(JNIEnv_*, const char*);
        return reinterpret_cast<fn>(functions->slot[6])(this, name);
    }
    jint Throw(jthrowable t)
    {
        typedef jint (*fn)(JNIEnv_*, jthrowable);
        return reinterpret_cast<fn>(functions->slot[13])(this, t);
    }
    jmethodID GetMethodID(jclass c, const char* name, const char* sig)
    {
        typedef jmethodID (*fn)(JNIEnv_*, jclass, const char*, const char*);
        return reinterpret_cast<fn>(functions->slot[33])(this, c, name, sig);
    }
    jobject NewObject(jclass c, jmethodID m, ...)
    {
        typedef jobject (*fn)(JNIEnv_*, jclass, jmethodID, va_list);
        va_list ap;
        va_start(ap, m);
        jobject o = reinterpret_cast<fn>(functions->slot[29])(this, c, m, ap);  /* NewObjectV */
        va_end(ap);
        return o;
    }
    jstring NewStringUTF(const char* s)
    {
        typedef jstring (*fn)(JNIEnv_*, const char*);
        return reinterpret_cast<fn>(functions->slot[167])(this, s);
    }
    void GetLongArrayRegion(jlongArray a, jsize start, jsize len, jlong* buf)
    {
        typedef void (*fn)(JNIEnv_*, jlongArray, jsize, jsize, jlong*);
        reinterpret_cast<fn>(functions->slot[204])(this, a, start, len, buf);
    }
};
typedef JNIEnv_ JNIEnv;
#endif
